// Linear ("lightning") attention with a per-head decay, as a recurrence over a per-request state.
//
// Per head, with q_t, k_t (D features) and v_t (Dv features), all after silu:
//     S_t = decay * S_{t-1} + k_t v_t^T            (S: [D, Dv] float32, zero at the start of a request)
//     o_t = S_t^T q_t
// The recurrence runs in float32 whatever the run type: the state, the decay, the outer product and the read-out.
// The projections arrive as rows of a fused matrix product (q columns, then k, then v; further columns, e.g. a
// gate's, may follow) in the run type; silu is applied as they are read (float32).
//
// One kernel serves prompt portions and single tokens.  The columns of S are independent, so a block owns
// (segment, head, a group of value columns) and walks the segment's tokens in order; a column's D state values
// are spread over L lanes (L a power of two, 16 values in registers per lane, zeros behind D), the read-out is
// summed over those lanes by shuffles.  The tokens' q, k and v are staged through shared memory a tile at a time.
// The state is stored [slot][head][value column][feature] so that a lane's values are contiguous.
//
// gated_rmsnorm: y = (o / sqrt(mean(o^2) + eps)) * w * sigmoid(g) over the concatenated heads of a token, the
// norm in float32; g are columns of the same fused projection.
#include <math.h>

#include "common.cuh"

#define LT_THREADS 128
#define LT_PER_LANE 16

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

template <typename T, int L>
__global__ void __launch_bounds__(LT_THREADS)
lightning_kernel(const T* __restrict__ proj, int row_stride, float* __restrict__ state, long long slot_stride,
                 const float* __restrict__ decay, const int* __restrict__ seg_start, const int* __restrict__ slots,
                 float* __restrict__ out, int H, int D, int Dv, int tile) {
    extern __shared__ __align__(16) float lt_smem[];
    constexpr int COLS = LT_THREADS / L;            // value columns of a block
    constexpr int DP = L * LT_PER_LANE;             // features of a head, padded to whole lanes (zeros behind D)
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int cw = threadIdx.x / L, part = threadIdx.x % L;
    const int col = c0 + cw;
    const int d0 = part * LT_PER_LANE;              // this lane's features d0 .. d0 + 15
    const bool live = col < Dv;
    const int t0 = seg_start[s], n = seg_start[s + 1] - t0;
    const float g = decay[h];
    float* st = state + (size_t)slots[s] * slot_stride + ((size_t)h * Dv + (live ? col : 0)) * D;
    float S[LT_PER_LANE];
#pragma unroll
    for (int i = 0; i < LT_PER_LANE; ++i) S[i] = (live && d0 + i < D) ? st[d0 + i] : 0.f;
    float* sq = lt_smem;                            // [tile][DP]
    float* sk = sq + (size_t)tile * DP;             // [tile][DP]
    float* sv = sk + (size_t)tile * DP;             // [tile][COLS]
    const int qo = h * D, ko = H * D + h * D, vo = 2 * H * D + h * Dv;
    for (int base = 0; base < n; base += tile) {
        const int m = min(tile, n - base);
        __syncthreads();
        for (int j = threadIdx.x; j < m * DP; j += LT_THREADS) {
            const int d = j % DP;
            const T* row = proj + (size_t)(t0 + base + j / DP) * row_stride;
            sq[j] = d < D ? silu_f(to_f32(row[qo + d])) : 0.f;
            sk[j] = d < D ? silu_f(to_f32(row[ko + d])) : 0.f;
        }
        for (int j = threadIdx.x; j < m * COLS; j += LT_THREADS) {
            const int c = c0 + j % COLS;
            sv[j] = c < Dv ? silu_f(to_f32(proj[(size_t)(t0 + base + j / COLS) * row_stride + vo + c])) : 0.f;
        }
        __syncthreads();
#pragma unroll 2
        for (int i = 0; i < m; ++i) {
            const float v = sv[i * COLS + cw];
            const float4* q4 = reinterpret_cast<const float4*>(sq + (size_t)i * DP + d0);
            const float4* k4 = reinterpret_cast<const float4*>(sk + (size_t)i * DP + d0);
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int r = 0; r < LT_PER_LANE / 4; ++r) {
                const float4 kk = k4[r], qq = q4[r];
                S[4 * r] = fmaf(g, S[4 * r], kk.x * v);
                S[4 * r + 1] = fmaf(g, S[4 * r + 1], kk.y * v);
                S[4 * r + 2] = fmaf(g, S[4 * r + 2], kk.z * v);
                S[4 * r + 3] = fmaf(g, S[4 * r + 3], kk.w * v);
                o0 = fmaf(S[4 * r], qq.x, o0);
                o1 = fmaf(S[4 * r + 1], qq.y, o1);
                o0 = fmaf(S[4 * r + 2], qq.z, o0);
                o1 = fmaf(S[4 * r + 3], qq.w, o1);
            }
            float o = o0 + o1;
#pragma unroll
            for (int x = L / 2; x > 0; x >>= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (part == 0 && live) out[(size_t)(t0 + base + i) * H * Dv + (size_t)h * Dv + col] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < LT_PER_LANE; ++i)
            if (d0 + i < D) st[d0 + i] = S[i];
    }
}

// The same walk for bfloat16 rows whose sizes allow 16-byte reads (D, Dv, the row stride and the columns of a block
// in multiples of 8, at most 256 features): the NEXT tile's q, k and v are requested into registers before the
// current tile's tokens are walked, so that the walk hides the latency of the reads (one long prompt gives a block
// per (head, column group) and nothing else on an SM to hide it).  Blocks of 32 or 64 threads (more blocks, fewer
// columns each) were measured and are slower: 766 against 434 us for 2,048 tokens of 16 heads of 64, since a
// block's four warps hide each other's shared-memory and shuffle latencies.
#define LT_FAST_ELEMS_PER_THREAD 32   // tile * DP / threads at most: q and k chunks of a tile are up to 4 + 4 reads of 16 bytes per thread
#define LT_FAST_TILE_MAX 64       // tokens of a tile at most (narrow heads)
#define LT_SLICE 20               // floats between the slices of two lanes in shared memory (16 used)

__device__ __forceinline__ void silu8_to_smem(const uint4& u, float* dst) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        dst[2 * i] = silu_f(__low2float(p[i]));
        dst[2 * i + 1] = silu_f(__high2float(p[i]));
    }
}

template <int L, int THREADS>
__global__ void __launch_bounds__(THREADS)
lightning_fast_kernel(const bf16* __restrict__ proj, int row_stride, float* __restrict__ state, long long slot_stride,
                      const float* __restrict__ decay, const int* __restrict__ seg_start, const int* __restrict__ slots,
                      float* __restrict__ out, int H, int D, int Dv) {
    extern __shared__ __align__(16) float lt_smem[];
    constexpr int COLS = THREADS / L;
    constexpr int DP = L * LT_PER_LANE;
    constexpr int ELEMS = LT_FAST_ELEMS_PER_THREAD * THREADS;
    constexpr int TILE = ELEMS / DP < LT_FAST_TILE_MAX ? ELEMS / DP : LT_FAST_TILE_MAX;
    constexpr int QK_CHUNKS = TILE * DP / 8;                  // 16-byte pieces of a tile's q (and of its k)
    constexpr int NPQ = QK_CHUNKS / THREADS;               // per thread: 4
    constexpr int V_CHUNKS = TILE * COLS / 8;
    constexpr int NPV = (V_CHUNKS + THREADS - 1) / THREADS;
    // a lane's 16 features lie LT_SLICE floats apart in shared memory: the lanes of a column then read their
    // 16-byte pieces from different banks (a stride of 16 floats would put every other lane on the same ones)
    constexpr int ROW = L * LT_SLICE;
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int cw = threadIdx.x / L, part = threadIdx.x % L;
    const int col = c0 + cw;
    const int d0 = part * LT_PER_LANE;
    const bool live = col < Dv;
    const int t0 = seg_start[s], n = seg_start[s + 1] - t0;
    const float g = decay[h];
    float* st = state + (size_t)slots[s] * slot_stride + ((size_t)h * Dv + (live ? col : 0)) * D;
    float S[LT_PER_LANE];
#pragma unroll
    for (int i = 0; i < LT_PER_LANE; ++i) S[i] = (live && d0 + i < D) ? st[d0 + i] : 0.f;
    float* sq = lt_smem;
    float* sk = sq + TILE * ROW;
    float* sv = sk + TILE * ROW;
    const int qo = h * D, ko = H * D + h * D, vo = 2 * H * D + h * Dv;
    uint4 pq[NPQ], pk[NPQ], pv[NPV];
    const uint4 zero = make_uint4(0, 0, 0, 0);
    auto request = [&](int base) {                            // the tile that starts at token `base` of the segment
        const int m = min(TILE, n - base);
#pragma unroll
        for (int p = 0; p < NPQ; ++p) {
            const int c = threadIdx.x + p * THREADS, tok = c / (DP / 8), d = (c % (DP / 8)) * 8;
            const bool on = tok < m && d < D;
            const bf16* row = proj + (size_t)(t0 + base + (on ? tok : 0)) * row_stride;
            pq[p] = on ? *reinterpret_cast<const uint4*>(row + qo + d) : zero;
            pk[p] = on ? *reinterpret_cast<const uint4*>(row + ko + d) : zero;
        }
#pragma unroll
        for (int p = 0; p < NPV; ++p) {
            const int c = threadIdx.x + p * THREADS, tok = c / (COLS / 8), cc = c0 + (c % (COLS / 8)) * 8;
            const bool on = c < V_CHUNKS && tok < m && cc < Dv;
            pv[p] = on ? *reinterpret_cast<const uint4*>(proj + (size_t)(t0 + base + tok) * row_stride + vo + cc) : zero;
        }
    };
    if (n > 0) request(0);
    for (int base = 0; base < n; base += TILE) {
        const int m = min(TILE, n - base);
        __syncthreads();                                      // the walk of the tile before is over
#pragma unroll
        for (int p = 0; p < NPQ; ++p) {                       // silu(0) = 0: padding stays zero
            const int c = threadIdx.x + p * THREADS, tok = c / (DP / 8), d = (c % (DP / 8)) * 8;
            const int at = tok * ROW + (d / LT_PER_LANE) * LT_SLICE + d % LT_PER_LANE;
            silu8_to_smem(pq[p], sq + at);
            silu8_to_smem(pk[p], sk + at);
        }
#pragma unroll
        for (int p = 0; p < NPV; ++p) {
            const int c = threadIdx.x + p * THREADS;
            if (c < V_CHUNKS) silu8_to_smem(pv[p], sv + (size_t)c * 8);
        }
        __syncthreads();
        if (base + TILE < n) request(base + TILE);            // in flight while this tile is walked
#pragma unroll 2
        for (int i = 0; i < m; ++i) {
            const float v = sv[i * COLS + cw];
            const float4* q4 = reinterpret_cast<const float4*>(sq + i * ROW + part * LT_SLICE);
            const float4* k4 = reinterpret_cast<const float4*>(sk + i * ROW + part * LT_SLICE);
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int r = 0; r < LT_PER_LANE / 4; ++r) {
                const float4 kk = k4[r], qq = q4[r];
                S[4 * r] = fmaf(g, S[4 * r], kk.x * v);
                S[4 * r + 1] = fmaf(g, S[4 * r + 1], kk.y * v);
                S[4 * r + 2] = fmaf(g, S[4 * r + 2], kk.z * v);
                S[4 * r + 3] = fmaf(g, S[4 * r + 3], kk.w * v);
                o0 = fmaf(S[4 * r], qq.x, o0);
                o1 = fmaf(S[4 * r + 1], qq.y, o1);
                o0 = fmaf(S[4 * r + 2], qq.z, o0);
                o1 = fmaf(S[4 * r + 3], qq.w, o1);
            }
            float o = o0 + o1;
#pragma unroll
            for (int x = L / 2; x > 0; x >>= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (part == 0 && live) out[(size_t)(t0 + base + i) * H * Dv + (size_t)h * Dv + col] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < LT_PER_LANE; ++i)
            if (d0 + i < D) st[d0 + i] = S[i];
    }
}

// proj [n_tokens, row_stride] of `dtype`: q at column 0 (H * D), k at H * D, v at 2 * H * D (H * Dv).  state: this
// layer's view, slot s at state + s * slot_stride floats, [H][Dv][D].  decay [H] float32.  out [n_tokens, H * Dv] float32.
GESSO_API int gesso_lightning(const void* proj, int dtype, int row_stride, float* state, long long slot_stride,
                              const float* decay, const int* seg_start, const int* slots, float* out, int n_tokens,
                              int n_segs, int H, int D, int Dv, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segs <= 0) return 0;
    if (H <= 0 || D <= 0 || Dv <= 0 || D > 32 * LT_PER_LANE || H > 65535 || row_stride < 2 * H * D + H * Dv)
        return GESSO_ERR_BAD_SIZE;
    int L = 1;
    while (L * LT_PER_LANE < D) L <<= 1;
    const int cols = LT_THREADS / L;
    if ((Dv + cols - 1) / cols > 65535) return GESSO_ERR_BAD_SIZE;
    const int dp = L * LT_PER_LANE;
    if (dtype == GESSO_BF16 && L <= 16 && D % 8 == 0 && Dv % 8 == 0 && row_stride % 8 == 0 && ((size_t)proj & 15) == 0) {
        const int threads = LT_THREADS;
        const int fcols = threads / L;
        const int elems = LT_FAST_ELEMS_PER_THREAD * threads;
        const int ftile = elems / dp < LT_FAST_TILE_MAX ? elems / dp : LT_FAST_TILE_MAX;
        const size_t fsmem = (size_t)ftile * (2 * L * LT_SLICE + fcols) * sizeof(float);
        const dim3 fgrid(n_segs, H, (Dv + fcols - 1) / fcols);
#define FGO(LL, TH)                                                                                                \
    do {                                                                                                           \
        static bool configured = false;   /* once per instantiation, outside any stream capture */                 \
        if (!configured) {                                                                                         \
            cudaFuncSetAttribute(lightning_fast_kernel<LL, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                 64 * 1024);                                                                       \
            configured = true;                                                                                     \
        }                                                                                                          \
        launch_pdl(lightning_fast_kernel<LL, TH>, fgrid, dim3(TH), fsmem, stream, (const bf16*)proj, row_stride,   \
                   state, slot_stride, decay, seg_start, slots, out, H, D, Dv);                                    \
    } while (0)
        switch (L) {
            case 1: FGO(1, 128); break;
            case 2: FGO(2, 128); break;
            case 4: FGO(4, 128); break;
            case 8: FGO(8, 128); break;
            default: FGO(16, 128); break;
        }
#undef FGO
        return launch_status();
    }
    int tile = 32;
    while (tile > 1 && (size_t)tile * (2 * dp + cols) * sizeof(float) > 44 * 1024) tile >>= 1;
    const size_t smem = (size_t)tile * (2 * dp + cols) * sizeof(float);
    const dim3 grid(n_segs, H, (Dv + cols - 1) / cols);
#define GO(T, LL)                                                                                                  \
    launch_pdl(lightning_kernel<T, LL>, grid, dim3(LT_THREADS), smem, stream, (const T*)proj, row_stride, state,   \
               slot_stride, decay, seg_start, slots, out, H, D, Dv, tile)
#define BY_L(T)                                                                                                    \
    switch (L) {                                                                                                   \
        case 1: GO(T, 1); break;                                                                                   \
        case 2: GO(T, 2); break;                                                                                   \
        case 4: GO(T, 4); break;                                                                                   \
        case 8: GO(T, 8); break;                                                                                   \
        case 16: GO(T, 16); break;                                                                                 \
        default: GO(T, 32); break;                                                                                 \
    }
    if (dtype == GESSO_F32) { BY_L(float) }
    else if (dtype == GESSO_BF16) { BY_L(bf16) }
    else return GESSO_ERR_BAD_DTYPE;
#undef BY_L
#undef GO
    return launch_status();
}

// ---- norm over the concatenated heads, times sigmoid(gate) ------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, const T* __restrict__ gate,
                     int gate_stride, T* __restrict__ out, int n_rows, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const float* row = o + (size_t)r * W;
    float ss = 0.f;
    for (int j = lane; j < W; j += 32) ss += row[j] * row[j];
    ss = warp_sum(ss);
    const float denom = sqrtf(ss / (float)W + eps);
    const T* g = gate + (size_t)r * gate_stride;
    for (int j = lane; j < W; j += 32) {
        const float sg = 1.f / (1.f + expf(-to_f32(g[j])));
        out[(size_t)r * W + j] = from_f32<T>((row[j] / denom) * w[j] * sg);
    }
}

// o [n_rows, W] float32; w [W] float32; gate: [n_rows, gate_stride] of `dtype` (the W gate columns at gate);
// out [n_rows, W] of `dtype`.
GESSO_API int gesso_gated_rmsnorm(const float* o, const float* w, float eps, const void* gate, int gate_stride,
                                  void* out, int dtype, int n_rows, int W, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (W <= 0 || gate_stride < W) return GESSO_ERR_BAD_SIZE;
    const dim3 grid((n_rows + 3) / 4);
    if (dtype == GESSO_F32)
        launch_pdl(gated_rmsnorm_kernel<float>, grid, dim3(128), 0, stream, o, w, eps, (const float*)gate, gate_stride,
                   (float*)out, n_rows, W);
    else if (dtype == GESSO_BF16)
        launch_pdl(gated_rmsnorm_kernel<bf16>, grid, dim3(128), 0, stream, o, w, eps, (const bf16*)gate, gate_stride,
                   (bf16*)out, n_rows, W);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}

// ---- prompt portions by chunks ------------------------------------------------------------------------------------
// The recurrence over a long portion, cut into the step's 64-token query tiles (a tile never crosses a request), so
// that the tiles run side by side instead of token after token.  With g the head's decay, a tile of m tokens that
// starts from the state S0 gives
//     o_t = g^(t+1) S0^T q_t + sum_{s <= t} g^(t-s) (q_t . k_s) v_s          (t = 0 .. m-1 inside the tile)
//     S_m = g^m S0 + U,   U = sum_s g^(m-1-s) k_s v_s^T
// Three launches: (1) every tile's U, from its own keys and values; (2) per (request, head) a walk over the request's
// tiles that turns the workspace's U into the state each tile starts from and leaves the last state in the slot;
// (3) every tile's outputs.  All float32 on the CUDA cores (4 x 4 register tiles over shared memory); the sums are
// the recurrence's own terms in another order.  The workspace holds one state [Dv][D] per (tile, head).
// A padded step repeats a tile at the end of its list; only a tile's first occurrence works.
#define LC_CHUNK 64
#define LC_THREADS 256

__device__ __forceinline__ float pow_int(float lg, int e) { return e == 0 ? 1.f : exp2f(lg * (float)e); }

// the tile's place in its request's list of tiles, or -1 for a repeated tile
__device__ __forceinline__ bool lc_tile(const int* tile_seg, const int* tile_q0, const int* seg_start, int tile, int& seg,
                                        int& q0, int& t0, int& m) {
    seg = tile_seg[tile];
    q0 = tile_q0[tile];
    const int first = tile - q0 / LC_CHUNK;
    if (first < 0 || tile_seg[first] != seg || tile_q0[first] != 0 || (first > 0 && tile_seg[first - 1] == seg)) return false;
    t0 = seg_start[seg];
    const int n = seg_start[seg + 1] - t0;
    if (q0 >= n) return false;
    m = min(LC_CHUNK, n - q0);
    return true;
}

template <typename T>
__global__ void __launch_bounds__(LC_THREADS)
lightning_chunk_state_kernel(const T* __restrict__ proj, int row_stride, const float* __restrict__ decay,
                             const int* __restrict__ seg_start, const int* __restrict__ tile_seg,
                             const int* __restrict__ tile_q0, float* __restrict__ ws, int H, int D, int Dv) {
    extern __shared__ __align__(16) float lc_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x, h = blockIdx.y;
    int seg, q0, t0, m;
    if (!lc_tile(tile_seg, tile_q0, seg_start, tile, seg, q0, t0, m)) return;
    const int DP = (D + 3) & ~3, VP = (Dv + 3) & ~3;
    float* sk = lc_smem;                    // [LC_CHUNK][DP], rows already weighted by g^(m-1-s)
    float* sv = sk + LC_CHUNK * DP;         // [LC_CHUNK][VP]
    const float lg = log2f(decay[h]);
    const int ko = H * D + h * D, vo = 2 * H * D + h * Dv;
    for (int j = threadIdx.x; j < LC_CHUNK * DP; j += LC_THREADS) {
        const int s = j / DP, d = j % DP;
        sk[j] = (s < m && d < D) ? silu_f(to_f32(proj[(size_t)(t0 + q0 + s) * row_stride + ko + d])) * pow_int(lg, m - 1 - s) : 0.f;
    }
    for (int j = threadIdx.x; j < LC_CHUNK * VP; j += LC_THREADS) {
        const int s = j / VP, c = j % VP;
        sv[j] = (s < m && c < Dv) ? silu_f(to_f32(proj[(size_t)(t0 + q0 + s) * row_stride + vo + c])) : 0.f;
    }
    __syncthreads();
    float* out = ws + ((size_t)tile * H + h) * Dv * D;
    const int dg_n = DP / 4, vg_n = VP / 4;
    for (int e = threadIdx.x; e < dg_n * vg_n; e += LC_THREADS) {
        const int dg = e % dg_n, vg = e / dg_n;
        float acc[4][4] = {};
        for (int s = 0; s < m; ++s) {
            const float4 kk = *reinterpret_cast<const float4*>(sk + s * DP + 4 * dg);
            const float4 vv = *reinterpret_cast<const float4*>(sv + s * VP + 4 * vg);
            const float ka[4] = {kk.x, kk.y, kk.z, kk.w}, va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(va[a], ka[b], acc[a][b]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (4 * vg + a < Dv && 4 * dg + b < D) out[(size_t)(4 * vg + a) * D + 4 * dg + b] = acc[a][b];
    }
}

__global__ void __launch_bounds__(LC_THREADS)
lightning_chunk_scan_kernel(float* __restrict__ state, long long slot_stride, const float* __restrict__ decay,
                            const int* __restrict__ seg_start, const int* __restrict__ slots,
                            const int* __restrict__ tile_seg, const int* __restrict__ tile_q0, int n_tiles,
                            float* __restrict__ ws, int H, int D, int Dv) {
    __shared__ int s_first;
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.x, h = blockIdx.y;
    if (threadIdx.x == 0) {
        int f = -1;
        for (int t = 0; t < n_tiles; ++t)
            if (tile_seg[t] == seg && tile_q0[t] == 0) { f = t; break; }
        s_first = f;
    }
    __syncthreads();
    const int first = s_first;
    const int e = blockIdx.z * LC_THREADS + threadIdx.x;
    if (first < 0 || e >= D * Dv) return;
    const int n = seg_start[seg + 1] - seg_start[seg];
    const float lg = log2f(decay[h]);
    float* st = state + (size_t)slots[seg] * slot_stride + (size_t)h * Dv * D + e;
    float S = *st;
    for (int c = 0; c * LC_CHUNK < n; ++c) {
        float* u = ws + ((size_t)(first + c) * H + h) * Dv * D + e;
        const float U = *u;
        *u = S;                                             // the state this tile starts from
        S = fmaf(pow_int(lg, min(LC_CHUNK, n - c * LC_CHUNK)), S, U);
    }
    *st = S;
}

template <typename T>
__global__ void __launch_bounds__(LC_THREADS)
lightning_chunk_out_kernel(const T* __restrict__ proj, int row_stride, const float* __restrict__ decay,
                           const int* __restrict__ seg_start, const int* __restrict__ tile_seg,
                           const int* __restrict__ tile_q0, const float* __restrict__ ws, float* __restrict__ out,
                           int H, int D, int Dv) {
    extern __shared__ __align__(16) float lc_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x, h = blockIdx.y;
    int seg, q0, t0, m;
    if (!lc_tile(tile_seg, tile_q0, seg_start, tile, seg, q0, t0, m)) return;
    const int DP = (D + 3) & ~3, VP = (Dv + 3) & ~3;
    const int WP = DP > VP ? DP : VP;
    float* sq = lc_smem;                        // [LC_CHUNK][DP]
    float* sx = sq + LC_CHUNK * DP;             // [LC_CHUNK][WP]: the keys, later the values
    float* sa = sx + LC_CHUNK * WP;             // [LC_CHUNK][LC_CHUNK + 4]: decayed scores, row t, column s
    constexpr int AP = LC_CHUNK + 4;
    const float lg = log2f(decay[h]);
    const int qo = h * D, ko = H * D + h * D, vo = 2 * H * D + h * Dv;
    for (int j = threadIdx.x; j < LC_CHUNK * DP; j += LC_THREADS) {
        const int s = j / DP, d = j % DP;
        const bool on = s < m && d < D;
        const T* row = proj + (size_t)(t0 + q0 + (on ? s : 0)) * row_stride;
        sq[j] = on ? silu_f(to_f32(row[qo + d])) : 0.f;
        sx[s * WP + d] = on ? silu_f(to_f32(row[ko + d])) : 0.f;
    }
    __syncthreads();
    // scores: 4 x 4 tiles of (t, s); above the diagonal they are zero
    for (int e = threadIdx.x; e < (LC_CHUNK / 4) * (LC_CHUNK / 4); e += LC_THREADS) {
        const int tg = e / (LC_CHUNK / 4), sg = e % (LC_CHUNK / 4);
        float acc[4][4] = {};
        if (sg <= tg) {
            for (int d = 0; d < DP; d += 4) {
                float4 qa[4], ka[4];
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    qa[a] = *reinterpret_cast<const float4*>(sq + (4 * tg + a) * DP + d);
                    ka[a] = *reinterpret_cast<const float4*>(sx + (4 * sg + a) * WP + d);
                }
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                        acc[a][b] += qa[a].x * ka[b].x + qa[a].y * ka[b].y + qa[a].z * ka[b].z + qa[a].w * ka[b].w;
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int t = 4 * tg + a, s = 4 * sg + b;
                sa[t * AP + s] = s <= t ? acc[a][b] * pow_int(lg, t - s) : 0.f;
            }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < LC_CHUNK * VP; j += LC_THREADS) {         // the values take the keys' place
        const int s = j / VP, c = j % VP;
        sx[s * WP + c] = (s < m && c < Dv) ? silu_f(to_f32(proj[(size_t)(t0 + q0 + s) * row_stride + vo + c])) : 0.f;
    }
    __syncthreads();
    const float* S0 = ws + ((size_t)tile * H + h) * Dv * D;                   // [Dv][D], the state the tile starts from
    const int vg_n = VP / 4;
    for (int e = threadIdx.x; e < (LC_CHUNK / 4) * vg_n; e += LC_THREADS) {
        const int tg = e / vg_n, vg = e % vg_n;
        float acc[4][4] = {};                                               // [t][v]
        for (int s = 0; s < 4 * tg + 4 && s < m; ++s) {
            const float4 vv = *reinterpret_cast<const float4*>(sx + s * WP + 4 * vg);
            const float va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float w = sa[(4 * tg + a) * AP + s];
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(w, va[b], acc[a][b]);
            }
        }
        // the carried state: g^(t+1) * sum_d q_t[d] S0[v][d]
        float car[4][4] = {};
        if ((D & 3) == 0) {
            // four features at a time: the state's rows are read as 16-byte pieces, several of them in flight
#pragma unroll 2
            for (int d = 0; d < D; d += 4) {
                float4 sv4[4], qv4[4];
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    sv4[b] = 4 * vg + b < Dv ? __ldg(reinterpret_cast<const float4*>(S0 + (size_t)(4 * vg + b) * D + d))
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int a = 0; a < 4; ++a) qv4[a] = *reinterpret_cast<const float4*>(sq + (4 * tg + a) * DP + d);
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                        car[a][b] += qv4[a].x * sv4[b].x + qv4[a].y * sv4[b].y + qv4[a].z * sv4[b].z + qv4[a].w * sv4[b].w;
            }
        } else {
            for (int d = 0; d < D; ++d) {
                float sv4[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) sv4[b] = 4 * vg + b < Dv ? S0[(size_t)(4 * vg + b) * D + d] : 0.f;
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    const float qv = sq[(4 * tg + a) * DP + d];
#pragma unroll
                    for (int b = 0; b < 4; ++b) car[a][b] = fmaf(qv, sv4[b], car[a][b]);
                }
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int t = 4 * tg + a;
            if (t >= m) continue;
            const float gt = pow_int(lg, t + 1);
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (4 * vg + b < Dv)
                    out[(size_t)(t0 + q0 + t) * H * Dv + (size_t)h * Dv + 4 * vg + b] = fmaf(gt, car[a][b], acc[a][b]);
        }
    }
}

// Bytes of workspace for a step of n_tiles query tiles.
GESSO_API long long gesso_lightning_chunked_workspace(int n_tiles, int H, int D, int Dv) {
    return (long long)n_tiles * H * D * Dv * (long long)sizeof(float);
}

GESSO_API int gesso_lightning_chunked_takes(int D, int Dv) { return D >= 1 && D <= 128 && Dv >= 1 && Dv <= 128; }

// The same arguments and result as gesso_lightning for a step with prompt portions; tile_seg / tile_q0 [n_tiles]: the step's
// 64-token query tiles; ws: gesso_lightning_chunked_workspace bytes.
GESSO_API int gesso_lightning_chunked(const void* proj, int dtype, int row_stride, float* state, long long slot_stride,
                                      const float* decay, const int* seg_start, const int* slots, const int* tile_seg,
                                      const int* tile_q0, int n_tiles, float* ws, float* out, int n_tokens, int n_segs,
                                      int H, int D, int Dv, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segs <= 0 || n_tiles <= 0) return 0;
    if (!gesso_lightning_chunked_takes(D, Dv) || H <= 0 || H > 65535 || n_segs > 65535 || row_stride < 2 * H * D + H * Dv)
        return GESSO_ERR_BAD_SIZE;
    const int DP = (D + 3) & ~3, VP = (Dv + 3) & ~3, WP = DP > VP ? DP : VP;
    const size_t smem_a = (size_t)LC_CHUNK * (DP + VP) * sizeof(float);
    const size_t smem_c = (size_t)LC_CHUNK * (DP + WP + LC_CHUNK + 4) * sizeof(float);
    const dim3 tiles(n_tiles, H), scan(n_segs, H, (D * Dv + LC_THREADS - 1) / LC_THREADS);
#define GO(T)                                                                                                          \
    do {                                                                                                               \
        static bool configured = false;   /* once per instantiation, outside any stream capture */                     \
        if (!configured) {                                                                                             \
            cudaFuncSetAttribute(lightning_chunk_state_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
            cudaFuncSetAttribute(lightning_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);   \
            configured = true;                                                                                         \
        }                                                                                                              \
        launch_pdl(lightning_chunk_state_kernel<T>, tiles, dim3(LC_THREADS), smem_a, stream, (const T*)proj, row_stride, \
                   decay, seg_start, tile_seg, tile_q0, ws, H, D, Dv);                                                 \
        launch_pdl(lightning_chunk_scan_kernel, scan, dim3(LC_THREADS), 0, stream, state, slot_stride, decay,          \
                   seg_start, slots, tile_seg, tile_q0, n_tiles, ws, H, D, Dv);                                        \
        launch_pdl(lightning_chunk_out_kernel<T>, tiles, dim3(LC_THREADS), smem_c, stream, (const T*)proj, row_stride, \
                   decay, seg_start, tile_seg, tile_q0, (const float*)ws, out, H, D, Dv);                              \
    } while (0)
    if (dtype == GESSO_F32) GO(float);
    else if (dtype == GESSO_BF16) GO(bf16);
    else return GESSO_ERR_BAD_DTYPE;
#undef GO
    return launch_status();
}
