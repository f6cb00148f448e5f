// Routed feed-forward for steps of many rows, grouped by expert, on the 5th-generation tensor cores.
//
//   1. moe_group_rows   counts the (token, expert) pairs of every expert, lays the experts out one after
//                       the other, each padded to whole 128-row tiles, and gives every pair its row; it also
//                       writes which expert each 128-row tile belongs to and how many tiles there are.
//   2. moe_gather_rows  copies every pair's input row to its place (bfloat16 [rows, K]).
//   3. moe_gemm_tcgen05 C[tile rows, N] = A[tile rows, K] * W[expert of the tile][N, K]^T for every tile: the
//                       same pipeline as the dense product of this library (TMA with 128-byte swizzle into a
//                       ring of stages, one thread issuing tcgen05.mma with float32 accumulators in tensor
//                       memory, double-buffered accumulators, four epilogue warps reading them back with
//                       tcgen05.ld); the only differences are that a tile's W rows start at
//                       expert * N + n0 of the stacked matrix [E * N, K] and that the number of row tiles is
//                       read from device memory (it depends on the routing; the grid is sized for the most
//                       there can be).  Epilogues: act(C) as bfloat16 (the up projection) or C as float32.
//   4. moe_combine      y[token] = sum_k weight_k * C[row of pair (token, k)], in the order of the choice.
//
// Rows of a tile beyond the expert's pairs are padding: they are computed from whatever the workspace
// holds and never read.  Every wait on an mbarrier is bounded and reports to the status word, as in the
// dense product.
#include <math.h>

#include "tcgen05.cuh"
#include "gemm_tcgen05_epilogue.cuh"
#include "tensor_map.cuh"

#define MG_BM 128
#define MG_BK 64
#define MG_THREADS 192

enum { MG_EPI_ACT_BF16 = 0, MG_EPI_F32 = 1, MG_EPI_GLU_BF16 = 2 };
enum { MG_ACT_RELU2 = 0, MG_ACT_SILU = 1, MG_ACT_GELU_TANH = 2 };
#define MG_GLU_ALPHA 1.702f

// A gated unit with clamped inputs on packed columns (8 gate columns, then their 8 up columns): 32 accumulator
// columns give 16 outputs, g * sigmoid(1.702 g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit);
// the output row is N / 2 wide.
__device__ __forceinline__ void mg_store_glu(const unsigned (&r)[32], void* __restrict__ out, int row, int col, int N,
                                             float limit) {
    bf16* o = reinterpret_cast<bf16*>(out) + (size_t)row * (N / 2) + col / 2;
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
        if (col + grp * 16 >= N) break;
        unsigned pk[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            float y[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const float g = fminf(__uint_as_float(r[grp * 16 + i + k]), limit);
                const float u = fminf(fmaxf(__uint_as_float(r[grp * 16 + 8 + i + k]), -limit), limit);
                y[k] = (g / (1.f + expf(-MG_GLU_ALPHA * g))) * (u + 1.f);
            }
            __nv_bfloat162 v = __floats2bfloat162_rn(y[0], y[1]);
            pk[i / 2] = *reinterpret_cast<unsigned*>(&v);
        }
        *reinterpret_cast<uint4*>(o + grp * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
}

__device__ __forceinline__ float mg_act(float v, int act) {
    if (act == MG_ACT_RELU2) { const float r = fmaxf(v, 0.f); return r * r; }
    if (act == MG_ACT_SILU) return v / (1.f + expf(-v));
    return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}

// ---- 1. rows by expert ------------------------------------------------------------------------------------
// top_idx [pairs]; pair_row [pairs] out; tile_expert [max tiles] out; counts_out[0] = tiles in use.
// One block; shared memory: 2 * E ints.
__global__ void __launch_bounds__(1024)
moe_group_rows_kernel(const int* __restrict__ top_idx, int n_pairs, int E, int* __restrict__ pair_row,
                      int* __restrict__ tile_expert, int* __restrict__ counts_out) {
    extern __shared__ int mg_smem[];
    int* count = mg_smem;          // pairs of every expert, then the cursor inside the expert's rows
    int* start = mg_smem + E;      // first row of every expert
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&count[top_idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0, tile = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = row;
            const int tiles = (count[e] + MG_BM - 1) / MG_BM;
            for (int i = 0; i < tiles; ++i) tile_expert[tile++] = e;
            row += tiles * MG_BM;
            count[e] = 0;
        }
        counts_out[0] = tile;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = top_idx[p];
        pair_row[p] = start[e] + atomicAdd(&count[e], 1);
    }
}

// ---- 2. input rows to their places ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const bf16* __restrict__ x, const int* __restrict__ pair_row, bf16* __restrict__ a, int n_pairs,
                       int top, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = K / 8;                                  // 16-byte pieces
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_pairs * per_row) return;
    const int p = (int)(idx / per_row), c = (int)(idx % per_row);
    const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)(p / top) * K + 8 * c);
    *reinterpret_cast<uint4*>(a + (size_t)pair_row[p] * K + 8 * c) = v;
}

// ---- 4. weighted sum of a token's experts ---------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ c, const int* __restrict__ pair_row, const float* __restrict__ top_w,
                   float* __restrict__ y, int n_tokens, int top, int N, int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = N / 4;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * per_row) return;
    const int t = (int)(idx / per_row), j = (int)(idx % per_row) * 4;
    float4 acc = accumulate ? *reinterpret_cast<const float4*>(y + (size_t)t * N + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    // eight experts at a time: their rows are looked up and requested together, then added in the order of the choice
    for (int k0 = 0; k0 < top; k0 += 8) {
        int row[8];
        float w[8];
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const bool on = k0 + i < top;
            row[i] = on ? pair_row[(size_t)t * top + k0 + i] : 0;
            w[i] = on ? top_w[(size_t)t * top + k0 + i] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            v[i] = k0 + i < top ? __ldcs(reinterpret_cast<const float4*>(c + (size_t)row[i] * N + j)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (k0 + i < top) { acc.x += w[i] * v[i].x; acc.y += w[i] * v[i].y; acc.z += w[i] * v[i].z; acc.w += w[i] * v[i].w; }
        }
    }
    *reinterpret_cast<float4*>(y + (size_t)t * N + j) = acc;
}

// ---- 3. the grouped product ------------------------------------------------------------------------------------
template <int BN, int STAGES>
struct __align__(1024) MgSmem {
    bf16 a[STAGES][MG_BM * MG_BK];
    bf16 b[STAGES][BN * MG_BK];
    unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    unsigned tmem_base;
};

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(MG_THREADS, 1)
moe_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        void* __restrict__ out, const int* __restrict__ tile_expert, const int* __restrict__ n_row_tiles,
                        int N, int K, int act, float limit, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    MgSmem<BN, STAGES>& s = *reinterpret_cast<MgSmem<BN, STAGES>*>(((size_t)smem_raw + 1023) & ~(size_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + MG_BK - 1) / MG_BK;
    const int n_blocks = (N + BN - 1) / BN;
    constexpr unsigned STAGE_BYTES = (MG_BM + BN) * MG_BK * sizeof(bf16);

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.acc_full[i], 1);
            mbar_init(&s.acc_empty[i], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(&s.tmem_base, 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = s.tmem_base;
    pdl_launch_dependents();
    pdl_wait();
    // how many row tiles the routing of this step made: every role walks the same list of tiles
    const int m_tiles = *n_row_tiles;
    const int n_tiles = m_tiles * n_blocks;

    if (warp == 0) {
        if (elect_one()) {
            unsigned it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int mt = tile % m_tiles, n0 = (tile / m_tiles) * BN;
                const int w_row = tile_expert[mt] * N + n0;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES;
                    const unsigned phase = (it / STAGES) & 1;
                    if (!mbar_wait(&s.empty[st], phase ^ 1)) { atomicExch(status, 2); ok = false; break; }
                    mbar_expect_tx(&s.full[st], STAGE_BYTES);
                    tma_load_2d(s.a[st], &map_a, kb * MG_BK, mt * MG_BM, &s.full[st]);
                    tma_load_2d(s.b[st], &map_w, kb * MG_BK, w_row, &s.full[st]);
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr unsigned idesc = make_idesc(MG_BM, BN);
            unsigned it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local) {
                const unsigned buf = local & 1;
                if (!mbar_wait(&s.acc_empty[buf], ((local >> 1) & 1) ^ 1)) { atomicExch(status, 5); ok = false; break; }
                tc_fence_after();
                const unsigned acc = tmem + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES;
                    const unsigned phase = (it / STAGES) & 1;
                    if (!mbar_wait(&s.full[st], phase)) { atomicExch(status, 3); ok = false; break; }
                    tc_fence_after();
                    const unsigned long long da = make_desc(smem_u32(s.a[st]));
                    const unsigned long long db = make_desc(smem_u32(s.b[st]));
#pragma unroll
                    for (int k = 0; k < MG_BK / 16; ++k)
                        umma_f16(acc, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&s.empty[st]);
                }
                umma_commit(&s.acc_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;
        unsigned local = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            const int mt = tile % m_tiles, n0 = (tile / m_tiles) * BN;
            const unsigned buf = local & 1;
            if (!mbar_wait(&s.acc_full[buf], (local >> 1) & 1)) {
                if (lane == 0) atomicExch(status, 4);
                break;
            }
            tc_fence_after();
            const int row = mt * MG_BM + q * 32 + lane;
            const unsigned acc = tmem + buf * BN + ((unsigned)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                unsigned r[32];
                tmem_ld32(acc + (unsigned)c, r);
                tmem_ld_wait();
                const int col = n0 + c;
                if (col >= N) continue;
                if (EPI == MG_EPI_GLU_BF16) {
                    mg_store_glu(r, out, row, col, N, limit);
                } else if (EPI == MG_EPI_ACT_BF16) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(mg_act(__uint_as_float(r[i]), act));
                    tc_store_32<TC_EPI_BF16>(r, out, nullptr, row, col, N);
                } else {
                    tc_store_32<TC_EPI_F32>(r, out, nullptr, row, col, N);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 2 * BN);
    }
}

// ---- host side ----------------------------------------------------------------------------------------------
// rows the workspace must hold for n_pairs pairs over E experts: every expert padded to whole tiles
GESSO_API long long gesso_moe_grouped_rows(long long n_pairs, int E) {
    const long long tiles = n_pairs / MG_BM + E;
    return tiles * MG_BM;
}

GESSO_API int gesso_moe_grouped_takes(int K, int F, int N) {
    // TMA: 16-byte rows (K % 8, F % 8); vector stores and the combine: F % 8, N % 8
    return K >= 8 && K % 8 == 0 && F >= 8 && F % 8 == 0 && N >= 8 && N % 8 == 0;
}

GESSO_API int gesso_moe_group_rows(const int* top_idx, int n_pairs, int E, int* pair_row, int* tile_expert,
                                   int* counts_out, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (E < 1 || E > 4096) return GESSO_ERR_BAD_SIZE;
    launch_pdl(moe_group_rows_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, top_idx, n_pairs, E,
               pair_row, tile_expert, counts_out);
    return launch_status();
}

GESSO_API int gesso_moe_gather_rows(const void* x, const int* pair_row, void* a, int n_pairs, int top, int K,
                                    cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (K % 8 != 0 || ((size_t)x & 15) || ((size_t)a & 15)) return GESSO_ERR_BAD_SIZE;
    const long long total = (long long)n_pairs * (K / 8);
    const long long blocks = (total + 255) / 256;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    launch_pdl(moe_gather_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)x, pair_row, (bf16*)a,
               n_pairs, top, K);
    return launch_status();
}

// accumulate: the sums are added to what y holds (a shared expert's output, say)
GESSO_API int gesso_moe_combine(const float* c, const int* pair_row, const float* top_w, float* y, int n_tokens, int top,
                                int N, int accumulate, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (N % 4 != 0) return GESSO_ERR_BAD_SIZE;
    const long long total = (long long)n_tokens * (N / 4);
    const long long blocks = (total + 255) / 256;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    launch_pdl(moe_combine_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, c, pair_row, top_w, y, n_tokens, top, N, accumulate);
    return launch_status();
}

template <int BN, int STAGES, int EPI>
static int launch_mg(const CUtensorMap& ma, const CUtensorMap& mw, void* out, const int* tile_expert, const int* n_row_tiles,
                     int max_row_tiles, int N, int K, int act, float limit, int* status, cudaStream_t stream) {
    const size_t smem = sizeof(MgSmem<BN, STAGES>) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(moe_gemm_tcgen05_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    const long long tiles = (long long)((N + BN - 1) / BN) * max_row_tiles;
    const int sms = gesso_sm_count();
    const dim3 grid((unsigned)(tiles < sms ? tiles : sms));
    launch_pdl(moe_gemm_tcgen05_kernel<BN, STAGES, EPI>, grid, dim3(MG_THREADS), smem, stream, ma, mw, out, tile_expert,
               n_row_tiles, N, K, act, limit, status);
    return launch_status();
}

// A: bfloat16 [rows_cap, K] (rows by expert, see moe_group_rows); W: bfloat16 [E, N, K]; out: [rows_cap, N],
// bfloat16 act(C) for epi 0, float32 C for epi 1; epi 2: bfloat16 [rows_cap, N / 2], the clamped gated unit on
// packed gate/up columns (N % 16 == 0).  tile_expert / n_row_tiles: from moe_group_rows, on the device.
GESSO_API int gesso_moe_gemm_tcgen05(const void* A, const void* W, void* out, const int* tile_expert,
                                     const int* n_row_tiles, long long rows_cap, int E, int N, int K, int epi, int act,
                                     float limit, int* status, cudaStream_t stream) {
    if (rows_cap <= 0) return 0;
    if (rows_cap % MG_BM != 0 || rows_cap > 2147483647LL || (long long)E * N > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (N < 8 || N % 8 != 0 || K < 8 || K % 8 != 0) return GESSO_ERR_BAD_SIZE;
    if (epi == MG_EPI_GLU_BF16 && N % 16 != 0) return GESSO_ERR_BAD_SIZE;
    if (((size_t)A & 15) || ((size_t)W & 15) || ((size_t)out & 15)) return GESSO_ERR_BAD_SIZE;
    const bool wide = N % 256 == 0 || N >= 1024;
    CUtensorMap ma, mw;
    int r = make_matrix_map(&ma, A, (int)rows_cap, K, MG_BM);
    if (r) return r;
    r = make_matrix_map(&mw, W, E * N, K, wide ? 256 : 128);
    if (r) return r;
    const int max_row_tiles = (int)(rows_cap / MG_BM);
#define GO(BN, ST)                                                                                                      \
    switch (epi) {                                                                                                      \
        case MG_EPI_ACT_BF16:                                                                                           \
            return launch_mg<BN, ST, MG_EPI_ACT_BF16>(ma, mw, out, tile_expert, n_row_tiles, max_row_tiles, N, K, act,  \
                                                      limit, status, stream);                                           \
        case MG_EPI_F32:                                                                                                \
            return launch_mg<BN, ST, MG_EPI_F32>(ma, mw, out, tile_expert, n_row_tiles, max_row_tiles, N, K, act,       \
                                                 limit, status, stream);                                                \
        case MG_EPI_GLU_BF16:                                                                                           \
            return launch_mg<BN, ST, MG_EPI_GLU_BF16>(ma, mw, out, tile_expert, n_row_tiles, max_row_tiles, N, K, act,  \
                                                      limit, status, stream);                                           \
        default: return GESSO_ERR_UNSUPPORTED;                                                                          \
    }
    if (wide) { GO(256, 4) } else { GO(128, 4) }
#undef GO
}
