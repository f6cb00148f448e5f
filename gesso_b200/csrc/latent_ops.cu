// Pieces of latent attention (queries and keys/values that go through a low-rank latent).
//
// 1. latent_norm_store: the fused down projection's rows p [N, Rq + Rkv] (float32 sums of a matrix product): the
//    first Rq columns are the query latent, the next Rkv the key/value latent.  Each piece is divided by its own
//    root mean square (eps inside the root) and scaled by its weight, in float32.  The query latent goes to
//    cq [N, Rq] (the operand of the up projection); the key/value latent c is the ONLY thing a position leaves in
//    the cache: it is written to the position's slot of the K pages ([page][1][slot][Rkv]).  Either piece may be
//    absent (Rq = 0: queries without a latent; write_kv = 0: an entry that reads another entry's cache).
//    With `v_pages` the latent is also written transposed ([page][1][Rkv][slot]), the layout from which the
//    tensor-core attention kernels read values; the token that ends a request's portion then zeroes the slots
//    behind its own up to the end of its 16-slot block (those kernels multiply masked weights, exact zeros, with
//    whatever such a slot holds, and pages pass from request to request as they are).  One warp per token.
//
// 2. headwise_linear: out[n, h, o] = sum_i W[h, i, o] x[n, h, i] for per-head matrices W [H, I, O] (input-major, so
//    that the threads of a block, one per output, read neighbouring elements).  Latent
//    attention in its absorbed form uses it twice: the query of head h is carried into the latent space,
//    q'[h] = W_uk[h]^T q[h] (so that scores are q' . c against the cached latent itself), and the weighted sum of
//    latents is carried out of it, o[h] = W_uv[h] (sum_j p_j c_j).  float32 accumulation; x, W and out each
//    float32 or bfloat16.  A block takes 4 rows x 1 head x 128 outputs; x rows sit in shared memory.
//
// 3. headwise_linear_tc: the same product on the tensor cores (mma.m16n8k16, bfloat16 in and out, float32
//    accumulation) for many rows, with the matrices output-major, W [H, O, I]: a block of four warps takes 64 rows x 1
//    head x 64 outputs, fragments read straight from global memory (the matrices are small and stay in L1/L2).
#include "common.cuh"

template <typename TO>
__global__ void __launch_bounds__(128)
latent_norm_store_kernel(const float* __restrict__ p, int Rq, int Rkv, const float* __restrict__ wq,
                         const float* __restrict__ wkv, float eps, TO* __restrict__ cq,
                         const int* __restrict__ positions, const int* __restrict__ seg_of_token,
                         const int* __restrict__ block_table, int max_pages, int page_size,
                         TO* __restrict__ k_pages, int write_kv, int* __restrict__ status, int n_tokens,
                         TO* __restrict__ v_pages) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const float* row = p + (size_t)t * (Rq + Rkv);
    if (Rq > 0) {
        float ss = 0.f;
        for (int j = lane; j < Rq; j += 32) ss += row[j] * row[j];
        ss = warp_sum(ss);
        const float denom = sqrtf(ss / (float)Rq + eps);
        for (int j = lane; j < Rq; j += 32) cq[(size_t)t * Rq + j] = from_f32<TO>((row[j] / denom) * wq[j]);
    }
    if (write_kv && Rkv > 0) {
        const float* r2 = row + Rq;
        float ss = 0.f;
        for (int j = lane; j < Rkv; j += 32) ss += r2[j] * r2[j];
        ss = warp_sum(ss);
        const float denom = sqrtf(ss / (float)Rkv + eps);
        const int pos = positions[t];
        const int page = block_table[(size_t)seg_of_token[t] * max_pages + pos / page_size];
        if (page < 0) {
            if (lane == 0) atomicExch(status, 1);
            return;
        }
        const int slot = pos % page_size;
        TO* dst = k_pages + ((size_t)page * page_size + slot) * Rkv;
        for (int j = lane; j < Rkv; j += 32) dst[j] = from_f32<TO>((r2[j] / denom) * wkv[j]);
        if (v_pages) {
            const bool last = t == n_tokens - 1 || seg_of_token[t + 1] != seg_of_token[t];
            const int clear = last ? min(page_size, ((slot >> 4) + 1) << 4) - slot : 1;
            TO* vt = v_pages + (size_t)page * Rkv * page_size + slot;
            for (int j = lane; j < Rkv; j += 32) {
                vt[(size_t)j * page_size] = from_f32<TO>((r2[j] / denom) * wkv[j]);
                for (int z = 1; z < clear; ++z) vt[(size_t)j * page_size + z] = from_f32<TO>(0.f);
            }
        }
    }
}

GESSO_API int gesso_latent_norm_store(const float* p, int Rq, int Rkv, const float* wq, const float* wkv, float eps,
                                      void* cq, int dtype, const int* positions, const int* seg_of_token,
                                      const int* block_table, int max_pages, int page_size, void* k_pages,
                                      int write_kv, int* status, int n_tokens, void* v_pages, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (Rq < 0 || Rkv < 0 || Rq + Rkv <= 0 || page_size <= 0) return GESSO_ERR_BAD_SIZE;
    const dim3 grid((n_tokens + 3) / 4);
    if (dtype == GESSO_F32)
        launch_pdl(latent_norm_store_kernel<float>, grid, dim3(128), 0, stream, p, Rq, Rkv, wq, wkv, eps, (float*)cq,
                   positions, seg_of_token, block_table, max_pages, page_size, (float*)k_pages, write_kv, status, n_tokens,
                   (float*)v_pages);
    else if (dtype == GESSO_BF16)
        launch_pdl(latent_norm_store_kernel<bf16>, grid, dim3(128), 0, stream, p, Rq, Rkv, wq, wkv, eps, (bf16*)cq,
                   positions, seg_of_token, block_table, max_pages, page_size, (bf16*)k_pages, write_kv, status, n_tokens,
                   (bf16*)v_pages);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}

// ---- per-head matrices ----------------------------------------------------------------------------------------
#define HW_ROWS 4
#define HW_OUTS 128

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(HW_OUTS)
headwise_linear_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out, int n_rows, int H,
                       int I, int O) {
    extern __shared__ float hw_x[];          // [HW_ROWS][I]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y, r0 = blockIdx.x * HW_ROWS, o = blockIdx.z * HW_OUTS + threadIdx.x;
    for (int j = threadIdx.x; j < HW_ROWS * I; j += HW_OUTS) {
        const int r = r0 + j / I;
        hw_x[j] = r < n_rows ? to_f32(x[((size_t)r * H + h) * I + (j % I)]) : 0.f;
    }
    __syncthreads();
    if (o >= O) return;
    const TW* wr = w + (size_t)h * I * O + o;
    float acc[HW_ROWS];
#pragma unroll
    for (int r = 0; r < HW_ROWS; ++r) acc[r] = 0.f;
    for (int i = 0; i < I; ++i) {
        const float wv = to_f32(wr[(size_t)i * O]);
#pragma unroll
        for (int r = 0; r < HW_ROWS; ++r) acc[r] += wv * hw_x[r * I + i];
    }
#pragma unroll
    for (int r = 0; r < HW_ROWS; ++r)
        if (r0 + r < n_rows) out[((size_t)(r0 + r) * H + h) * O + o] = from_f32<TO>(acc[r]);
}

// x [n_rows, H, I], w [H, I, O], out [n_rows, H, O]; dtypes each GESSO_F32 or GESSO_BF16.
GESSO_API int gesso_headwise_linear(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                                    int n_rows, int H, int I, int O, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || I <= 0 || O <= 0 || H > 65535 || (O + HW_OUTS - 1) / HW_OUTS > 65535) return GESSO_ERR_BAD_SIZE;
    const size_t smem = (size_t)HW_ROWS * I * sizeof(float);
    if (smem > 48 * 1024) return GESSO_ERR_BAD_SIZE;
    const dim3 grid((n_rows + HW_ROWS - 1) / HW_ROWS, H, (O + HW_OUTS - 1) / HW_OUTS);
#define GO(TX, TW, TO)                                                                                             \
    launch_pdl(headwise_linear_kernel<TX, TW, TO>, grid, dim3(HW_OUTS), smem, stream, (const TX*)x, (const TW*)w,  \
               (TO*)out, n_rows, H, I, O)
    const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (key) {
        case 0: GO(float, float, float); break;
        case 1: GO(float, float, bf16); break;
        case 2: GO(float, bf16, float); break;
        case 3: GO(float, bf16, bf16); break;
        case 4: GO(bf16, float, float); break;
        case 5: GO(bf16, float, bf16); break;
        case 6: GO(bf16, bf16, float); break;
        case 7: GO(bf16, bf16, bf16); break;
        default: return GESSO_ERR_BAD_DTYPE;
    }
#undef GO
    return launch_status();
}

// ---- the same on the tensor cores ------------------------------------------------------------------------------------
__device__ __forceinline__ void hw_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128)
headwise_linear_tc_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ out, int n_rows, int H,
                          int I, int O) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int h = blockIdx.y, r0 = blockIdx.x * 64 + 16 * warp, n0 = blockIdx.z * 64;
    if (r0 >= n_rows) return;
    // rows and outputs past the end repeat the last one (computed, never stored)
    const int ra = min(r0 + g, n_rows - 1), rb = min(r0 + g + 8, n_rows - 1);
    const bf16* xa = x + ((size_t)ra * H + h) * I + 2 * t;
    const bf16* xb = x + ((size_t)rb * H + h) * I + 2 * t;
    const bf16* wn[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) wn[j] = w + ((size_t)h * O + min(n0 + 8 * j + g, O - 1)) * I + 2 * t;
    float acc[8][4] = {};
    for (int k = 0; k < I; k += 16) {
        const unsigned a0 = *reinterpret_cast<const unsigned*>(xa + k), a1 = *reinterpret_cast<const unsigned*>(xb + k);
        const unsigned a2 = *reinterpret_cast<const unsigned*>(xa + k + 8), a3 = *reinterpret_cast<const unsigned*>(xb + k + 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const unsigned b0 = *reinterpret_cast<const unsigned*>(wn[j] + k), b1 = *reinterpret_cast<const unsigned*>(wn[j] + k + 8);
            hw_mma(acc[j], a0, a1, a2, a3, b0, b1);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int n = n0 + 8 * j + 2 * t;
        if (n >= O) continue;                     // O is even: n + 1 < O too
        if (r0 + g < n_rows)
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(r0 + g) * H + h) * O + n) = __floats2bfloat162_rn(acc[j][0], acc[j][1]);
        if (r0 + g + 8 < n_rows)
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(r0 + g + 8) * H + h) * O + n) = __floats2bfloat162_rn(acc[j][2], acc[j][3]);
    }
}

GESSO_API int gesso_headwise_linear_tc_takes(int I, int O) { return I >= 16 && I % 16 == 0 && O >= 8 && O % 8 == 0; }

// x [n_rows, H, I], w [H, O, I] (output-major), out [n_rows, H, O], all bfloat16.
GESSO_API int gesso_headwise_linear_tc(const void* x, const void* w, void* out, int n_rows, int H, int I, int O,
                                       cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!gesso_headwise_linear_tc_takes(I, O) || H <= 0 || H > 65535 || (O + 63) / 64 > 65535) return GESSO_ERR_BAD_SIZE;
    if (((size_t)x & 3) || ((size_t)w & 3) || ((size_t)out & 3)) return GESSO_ERR_BAD_SIZE;
    const dim3 grid((n_rows + 63) / 64, H, (O + 63) / 64);
    launch_pdl(headwise_linear_tc_kernel, grid, dim3(128), 0, stream, (const bf16*)x, (const bf16*)w, (bf16*)out, n_rows, H,
               I, O);
    return launch_status();
}
