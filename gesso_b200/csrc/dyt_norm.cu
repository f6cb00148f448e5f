// Dynamic Tanh norm with the residual add folded in.
//
// The norm computes no statistics: y = tanh(alpha * x) * w + b with a scalar alpha and vectors w, b.
// A layer that norms a sublayer's output before adding it ("post" norm) and norms the sum again for
// the next sublayer ("pre" norm) does both in this one pass over the float32 residual stream:
//
//     v      = h + post(delta)          post(d) = tanh(alpha_p * d) * w_p + b_p   (or d itself without a post norm)
//     h      = v                        (not with a row list: only the listed rows are computed, h stays)
//     out    = tanh(alpha * v) * w + b  (rounded to the run type; no output without a pre norm)
//
// Everything is float32 inside; tanhf is the accurate one.  One thread per four consecutive features
// (one feature where the width is not a multiple of four).
#include <math.h>

#include "common.cuh"

struct DytParams {
    float alpha;
    const float* w;   // null: this norm is absent
    const float* b;   // may be null (no shift)
};

__device__ __forceinline__ float dyt_apply(const DytParams& p, float x, int j) {
    return tanhf(p.alpha * x) * p.w[j] + (p.b ? p.b[j] : 0.f);
}

template <typename TD, typename TO, int VEC>
__global__ void __launch_bounds__(256)
add_dyt_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ delta_bias,
               DytParams post, DytParams pre, TO* __restrict__ out, const int* __restrict__ rows, long long n_out,
               int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = H / VEC;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_out * per_row) return;
    const long long i = idx / per_row;
    const int j0 = (int)(idx % per_row) * VEC;
    const long long r = rows ? rows[i] : i;
    float v[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = h[r * H + j0 + k];
    if (delta) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            float d = to_f32(delta[r * H + j0 + k]);
            if (delta_bias) d += delta_bias[j0 + k];
            v[k] += post.w ? dyt_apply(post, d, j0 + k) : d;
        }
        if (!rows) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) h[r * H + j0 + k] = v[k];
        }
    }
    if (pre.w) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) out[i * H + j0 + k] = from_f32<TO>(dyt_apply(pre, v[k], j0 + k));
    }
}

// h: float32 [N, H], updated in place unless `rows` is given.  delta: [N, H] of delta_dtype, or null.
// post_w / pre_w null: that norm is absent.  out: [n_out, H] of out_dtype (unused without a pre norm).
GESSO_API int gesso_add_dyt(float* h, const void* delta, int delta_dtype, const float* delta_bias, float post_alpha,
                            const float* post_w, const float* post_b, float pre_alpha, const float* pre_w,
                            const float* pre_b, void* out, int out_dtype, const int* rows, int n_out, int H,
                            cudaStream_t stream) {
    if (n_out <= 0 || H <= 0) return 0;
    if (!delta && !pre_w) return 0;
    const DytParams post = {post_alpha, post_w, post_b}, pre = {pre_alpha, pre_w, pre_b};
    const int vec = H % 4 == 0 ? 4 : 1;
    const long long total = (long long)n_out * (H / vec);
    const long long blocks = (total + 255) / 256;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
#define GO(TD, TO)                                                                                               \
    do {                                                                                                         \
        if (vec == 4)                                                                                            \
            launch_pdl(add_dyt_kernel<TD, TO, 4>, dim3((unsigned)blocks), dim3(256), 0, stream, h,               \
                       (const TD*)delta, delta_bias, post, pre, (TO*)out, rows, (long long)n_out, H);            \
        else                                                                                                     \
            launch_pdl(add_dyt_kernel<TD, TO, 1>, dim3((unsigned)blocks), dim3(256), 0, stream, h,               \
                       (const TD*)delta, delta_bias, post, pre, (TO*)out, rows, (long long)n_out, H);            \
    } while (0)
    const bool d16 = delta && delta_dtype == GESSO_BF16;
    if (delta && delta_dtype != GESSO_BF16 && delta_dtype != GESSO_F32) return GESSO_ERR_BAD_DTYPE;
    if (out_dtype == GESSO_BF16) {
        if (d16) GO(bf16, bf16); else GO(float, bf16);
    } else if (out_dtype == GESSO_F32) {
        if (d16) GO(bf16, float); else GO(float, float);
    } else {
        return GESSO_ERR_BAD_DTYPE;
    }
#undef GO
    return launch_status();
}
