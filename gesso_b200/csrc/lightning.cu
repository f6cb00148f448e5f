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
// are spread over L lanes (L a power of two, D / L <= 16 values in registers per lane), the read-out is summed
// over those lanes by shuffles.  The tokens' q, k and v are staged through shared memory a tile at a time.
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
    extern __shared__ float lt_smem[];
    constexpr int COLS = LT_THREADS / L;            // value columns of a block
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int col = c0 + threadIdx.x / L, part = threadIdx.x % L;
    const int per = (D + L - 1) / L;                // features of a lane (<= LT_PER_LANE)
    const int d0 = part * per;
    const bool live = col < Dv;
    const int t0 = seg_start[s], n = seg_start[s + 1] - t0;
    const float g = decay[h];
    float* st = state + (size_t)slots[s] * slot_stride + ((size_t)h * Dv + (live ? col : 0)) * D;
    float S[LT_PER_LANE];
#pragma unroll
    for (int i = 0; i < LT_PER_LANE; ++i) S[i] = (live && i < per && d0 + i < D) ? st[d0 + i] : 0.f;
    float* sq = lt_smem;                            // [tile][D]
    float* sk = sq + (size_t)tile * D;              // [tile][D]
    float* sv = sk + (size_t)tile * D;              // [tile][COLS]
    const int qo = h * D, ko = H * D + h * D, vo = 2 * H * D + h * Dv;
    for (int base = 0; base < n; base += tile) {
        const int m = min(tile, n - base);
        __syncthreads();
        for (int j = threadIdx.x; j < m * D; j += LT_THREADS) {
            const T* row = proj + (size_t)(t0 + base + j / D) * row_stride;
            sq[j] = silu_f(to_f32(row[qo + j % D]));
            sk[j] = silu_f(to_f32(row[ko + j % D]));
        }
        for (int j = threadIdx.x; j < m * COLS; j += LT_THREADS) {
            const int c = c0 + j % COLS;
            sv[j] = c < Dv ? silu_f(to_f32(proj[(size_t)(t0 + base + j / COLS) * row_stride + vo + c])) : 0.f;
        }
        __syncthreads();
        for (int i = 0; i < m; ++i) {
            const float v = sv[i * COLS + threadIdx.x / L];
            const float* qi = sq + (size_t)i * D + d0;
            const float* ki = sk + (size_t)i * D + d0;
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < LT_PER_LANE; ++r) {
                if (r < per && d0 + r < D) {
                    S[r] = fmaf(g, S[r], ki[r] * v);
                    o = fmaf(S[r], qi[r], o);
                }
            }
#pragma unroll
            for (int x = L / 2; x > 0; x >>= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (part == 0 && live) out[(size_t)(t0 + base + i) * H * Dv + (size_t)h * Dv + col] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < LT_PER_LANE; ++i)
            if (i < per && d0 + i < D) st[d0 + i] = S[i];
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
    int tile = 16;
    while (tile > 1 && (size_t)tile * (2 * D + cols) * sizeof(float) > 40 * 1024) tile >>= 1;
    const size_t smem = (size_t)tile * (2 * D + cols) * sizeof(float);
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
