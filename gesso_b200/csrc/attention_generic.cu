// Paged causal attention for any head size up to 512, in float32 arithmetic (CUDA cores).
//
// This is the kernel of the true 32-bit path, and the bfloat16 path uses it for head sizes its
// tensor-core kernels do not take.  One warp per (token, query head).  A query at absolute
// position p reads keys lo..p of its own request, lo = max(0, p - window + 1) with a window,
// else 0 (src/Inference/Inference.jl:1206-1207).  Query head h reads kv head h / (nh/nkv)
// (src/Inference/Inference.jl:1398).  Score = (q . k) / sqrt(hd); softmax and the weighted sum
// of values are float32 with a running maximum per lane (lanes stride over keys) that is
// merged across the warp at the end, so the result does not depend on which pages hold the keys
// or on what else is in the batch.
//
// Options, all off by default: values of another width than the keys (`vd`); a window that also keeps the
// first `keep_first` positions of the sequence visible (key u is read if u <= p and (p - u < window or
// u < keep_first)); a caller's scale instead of 1/sqrt(hd) (the scale is always passed in); an output gate:
// the result is multiplied by sigmoid(gate[t, h * vd + j]) before it is stored (`gate` rows are
// `gate_stride` elements apart, e.g. further columns of the fused projection); a learned sink per query head
// (`sink`: exp(sink[h]) is added to the softmax denominator: it takes weight away from every key and contributes
// nothing to the result; the score scale is not applied to it); a
// distance bias per query head (`slopes`: slopes[h] * (p - u) is taken off the score of key u); values that ARE
// the keys (`v_from_k`: the weighted sum runs over the key rows themselves, as latent attention in its absorbed
// form wants: one shared latent per position is key and value of every head); queries and results in float32
// over bfloat16 pages (`TQ` = float, `T` = bf16).
#include <math.h>

#include "common.cuh"

template <typename TQ, typename T, int HD_PAD>
__global__ void __launch_bounds__(128)
paged_attention_generic_kernel(const TQ* __restrict__ q, const T* __restrict__ k_pages,
                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                               int max_pages, int page_size, const int* __restrict__ positions,
                               const int* __restrict__ seg_of_token, TQ* __restrict__ out, int n_tokens,
                               int nh, int nkv, int hd, int window, float scale, int vd, int keep_first,
                               const T* __restrict__ gate, int gate_stride, const float* __restrict__ sink,
                               const float* __restrict__ slopes, int v_from_k) {
    __shared__ float q_s[4][HD_PAD];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long wi = (long long)blockIdx.x * 4 + wid;
    if (wi >= (long long)n_tokens * nh) return;   // whole warps leave together; no block barrier below
    const int t = (int)(wi / nh), h = (int)(wi % nh);
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int* bt = block_table + (size_t)seg_of_token[t] * max_pages;
    const TQ* qrow = q + ((size_t)t * nh + h) * hd;
    const float slope = slopes ? slopes[h] : 0.f;
    for (int j = lane; j < HD_PAD; j += 32) q_s[wid][j] = j < hd ? to_f32(qrow[j]) : 0.f;
    __syncwarp();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.f;
    float acc[HD_PAD];
#pragma unroll
    for (int j = 0; j < HD_PAD; ++j) acc[j] = 0.f;

    // with a window, the kept first positions come first (lanes stride over them), then the window itself
    const int n_kept = lo > 0 ? min(keep_first, lo) : 0;
    for (int uu = lane; uu < n_kept + (pos - lo + 1); uu += 32) {
        const int u = uu < n_kept ? uu : lo + (uu - n_kept);
        const int page = bt[u / page_size];
        if (page < 0) continue;
        const T* kr = k_pages + (((size_t)page * nkv + kvh) * page_size + (u % page_size)) * hd;
        // V is stored [feature][slot] inside a page
        const T* vr = v_from_k ? kr : v_pages + ((size_t)page * nkv + kvh) * vd * page_size + (u % page_size);
        const size_t v_step = v_from_k ? 1 : (size_t)page_size;
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < HD_PAD; ++j)
            if (j < hd) dot += q_s[wid][j] * to_f32(kr[j]);
        const float sc = dot * scale - slope * (float)(pos - u);
        if (sc > m) {
            const float corr = expf(m - sc);   // exp(-inf) = 0 on the first key
            l *= corr;
#pragma unroll
            for (int j = 0; j < HD_PAD; ++j) acc[j] *= corr;
            m = sc;
        }
        const float p = expf(sc - m);
        l += p;
#pragma unroll
        for (int j = 0; j < HD_PAD; ++j)
            if (j < vd) acc[j] += p * to_f32(vr[(size_t)j * v_step]);
    }
    float M = warp_max(m);
    if (sink) M = fmaxf(M, sink[h]);
    const float f = (m == -INFINITY) ? 0.f : expf(m - M);
    float L = warp_sum(l * f);
    if (sink) L += expf(sink[h] - M);                // the sink enters the denominator only
    TQ* orow = out + ((size_t)t * nh + h) * vd;
    const T* grow = gate ? gate + (size_t)t * gate_stride + (size_t)h * vd : nullptr;
#pragma unroll
    for (int j = 0; j < HD_PAD; ++j) {
        const float a = warp_sum(acc[j] * f);
        if (j < vd && (j & 31) == lane) {
            float y = a / L;
            if (grow) y *= 1.f / (1.f + expf(-to_f32(grow[j])));
            orow[j] = from_f32<TQ>(y);
        }
    }
}

template <typename TQ, typename T>
static int launch_generic(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                          int max_pages, int page_size, const int* positions, const int* seg_of_token,
                          void* out, int n_tokens, int nh, int nkv, int hd, int window, float scale, int vd,
                          int keep_first, const void* gate, int gate_stride, const float* sink, const float* slopes,
                          int v_from_k, cudaStream_t stream) {
    const long long total = (long long)n_tokens * nh;
    const long long blocks = (total + 3) / 4;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
#define GO(PAD)                                                                                          \
    paged_attention_generic_kernel<TQ, T, PAD><<<(unsigned)blocks, 128, 0, stream>>>(                     \
        (const TQ*)q, (const T*)k_pages, (const T*)v_pages, block_table, max_pages, page_size, positions, \
        seg_of_token, (TQ*)out, n_tokens, nh, nkv, hd, window, scale, vd, keep_first, (const T*)gate,     \
        gate_stride, sink, slopes, v_from_k)
    const int wide = hd > vd ? hd : vd;
    if (wide <= 32) GO(32);
    else if (wide <= 64) GO(64);
    else if (wide <= 128) GO(128);
    else if (wide <= 256) GO(256);
    else if (wide <= 512) GO(512);
    else return GESSO_ERR_BAD_SIZE;
#undef GO
    return launch_status();
}

// `q_dtype`: the type of q and of the result; `dtype`: the type of the pages (and of the gate).  A float32 q may
// read bfloat16 pages; otherwise the two are equal.
GESSO_API int gesso_paged_attention_generic(const void* q, const void* k_pages, const void* v_pages, int dtype,
                                            const int* block_table, int max_pages, int page_size,
                                            const int* positions, const int* seg_of_token, void* out,
                                            int n_tokens, int nh, int nkv, int hd, int window, float scale,
                                            int vd, int keep_first, const void* gate, int gate_stride,
                                            int q_dtype, const float* sink, const float* slopes, int v_from_k,
                                            cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0) return GESSO_ERR_BAD_SIZE;
    if (v_from_k) vd = hd;
    if (vd <= 0) vd = hd;
    if (keep_first < 0 || (gate && gate_stride < nh * vd)) return GESSO_ERR_BAD_SIZE;
#define ARGS q, k_pages, v_pages, block_table, max_pages, page_size, positions, seg_of_token, out, n_tokens, nh, nkv, hd, \
             window, scale, vd, keep_first, gate, gate_stride, sink, slopes, v_from_k, stream
    if (dtype == GESSO_F32 && q_dtype == GESSO_F32) return launch_generic<float, float>(ARGS);
    if (dtype == GESSO_BF16 && q_dtype == GESSO_BF16) return launch_generic<bf16, bf16>(ARGS);
    if (dtype == GESSO_BF16 && q_dtype == GESSO_F32) return launch_generic<float, bf16>(ARGS);
#undef ARGS
    return GESSO_ERR_BAD_DTYPE;
}
