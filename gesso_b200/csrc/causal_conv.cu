// A short causal convolution over time on every channel of a projection's rows, with a per-request state.
//
// The rows u [N, row_stride] come from a matrix product (C channels from column 0; a bias vector is added first,
// as the projection's own bias).  On the flat token axis of a step, token t of segment s at place i inside its
// portion gets
//     y[t, c] = sum_{j < L} taps[c, j] * u'(i - (L - 1) + j, c),      u' = u + bias,
// where places before the portion's start come from the request's state [L-1, C] (the last L-1 values of u' of
// earlier steps, oldest first; zeros at the start of a request because a fresh slot is zeroed; a single tap,
// L = 1, keeps no state).  Arithmetic is
// float32; the state is float32, so a cut between two steps is invisible to it.
//
// Optional value mixing on a column range of the OUTPUT: y[t, c] = (1 - lambda) * y[t, c] + lambda * first[t, c - c0]
// for c0 <= c < c0 + n_mix (`first` rows are `first_stride` elements apart): what an attention layer that mixes
// its values with an earlier layer's values of the same token needs right behind its convolution.
//
// Two launches: the convolution reads the old state, then a second kernel moves the state on (one thread per
// (segment, channel) reads what it needs before it writes), so no thread reads a state another has replaced.
#include "common.cuh"

#define CCONV_MAX_TAPS 8

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const T* __restrict__ u, int row_stride, const float* __restrict__ bias,
                   const float* __restrict__ taps, const float* __restrict__ state, long long slot_stride,
                   const int* __restrict__ seg_of_token, const int* __restrict__ seg_start,
                   const int* __restrict__ slots, T* __restrict__ out, int n_tokens, int C, int L,
                   const T* __restrict__ first, int first_stride, int mix_c0, int n_mix, float lambda) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * C) return;
    const int t = (int)(i / C), c = (int)(i % C);
    const int s = seg_of_token[t];
    const int place = t - seg_start[s];
    const float b = bias ? bias[c] : 0.f;
    const float* st = state + (size_t)slots[s] * slot_stride;
    float acc = 0.f;
    for (int j = 0; j < L; ++j) {
        const int src = place - (L - 1) + j;
        const float v = src >= 0 ? to_f32(u[(size_t)(t - place + src) * row_stride + c]) + b
                                 : st[(size_t)(L - 1 + src) * C + c];
        acc += taps[(size_t)c * L + j] * v;
    }
    if (first && c >= mix_c0 && c < mix_c0 + n_mix)
        acc = (1.f - lambda) * acc + lambda * to_f32(first[(size_t)t * first_stride + (c - mix_c0)]);
    out[(size_t)t * C + c] = from_f32<T>(acc);
}

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_state_kernel(const T* __restrict__ u, int row_stride, const float* __restrict__ bias,
                         float* __restrict__ state, long long slot_stride, const int* __restrict__ seg_start,
                         const int* __restrict__ slots, int n_segs, int C, int L) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_segs * C) return;
    const int s = (int)(i / C), c = (int)(i % C);
    const int t0 = seg_start[s], n = seg_start[s + 1] - t0;
    const float b = bias ? bias[c] : 0.f;
    float* st = state + (size_t)slots[s] * slot_stride;
    float keep[CCONV_MAX_TAPS - 1];
#pragma unroll
    for (int r = 0; r < CCONV_MAX_TAPS - 1; ++r) {
        if (r >= L - 1) break;
        const int src = n - (L - 1) + r;          // place inside the portion of the value that lands in row r
        keep[r] = src >= 0 ? to_f32(u[(size_t)(t0 + src) * row_stride + c]) + b : st[(size_t)(L - 1 + src) * C + c];
    }
#pragma unroll
    for (int r = 0; r < CCONV_MAX_TAPS - 1; ++r) {
        if (r >= L - 1) break;
        st[(size_t)r * C + c] = keep[r];
    }
}

// u [n_tokens, row_stride] and out [n_tokens, C] of `dtype`; bias [C] or null, taps [C, L] float32; state: this
// layer's view, slot s at state + s * slot_stride, [L-1, C] float32.  first: [n_tokens, first_stride] of `dtype` or null.
GESSO_API int gesso_causal_conv(const void* u, int dtype, int row_stride, const float* bias, const float* taps,
                                float* state, long long slot_stride, const int* seg_of_token, const int* seg_start,
                                const int* slots, void* out, int n_tokens, int n_segs, int C, int L,
                                const void* first, int first_stride, int mix_c0, int n_mix, float lambda,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (C <= 0 || L < 1 || L > CCONV_MAX_TAPS || row_stride < C || n_segs <= 0) return GESSO_ERR_BAD_SIZE;
    if (first && (mix_c0 < 0 || n_mix <= 0 || mix_c0 + n_mix > C || first_stride < n_mix)) return GESSO_ERR_BAD_SIZE;
    const long long total = (long long)n_tokens * C, blocks = (total + 255) / 256;
    const long long sblocks = ((long long)n_segs * C + 255) / 256;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
#define GO(T)                                                                                                        \
    do {                                                                                                             \
        launch_pdl(causal_conv_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (const T*)u, row_stride, bias, \
                   taps, (const float*)state, slot_stride, seg_of_token, seg_start, slots, (T*)out, n_tokens, C, L,  \
                   (const T*)first, first_stride, mix_c0, n_mix, lambda);                                            \
        if (L > 1)                                                                                                   \
            launch_pdl(causal_conv_state_kernel<T>, dim3((unsigned)sblocks), dim3(256), 0, stream, (const T*)u,      \
                       row_stride, bias, state, slot_stride, seg_start, slots, n_segs, C, L);                        \
    } while (0)
    if (dtype == GESSO_F32) GO(float);
    else if (dtype == GESSO_BF16) GO(bf16);
    else return GESSO_ERR_BAD_DTYPE;
#undef GO
    return launch_status();
}
