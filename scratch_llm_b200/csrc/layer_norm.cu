// Layer norm (mean and variance, gain and offset) fused with the add of what a layer left
// pending for the residual stream.
//
//   x[n]   = resid[n] + sum_i coef_i * term_i[n]          (up to LN_MAX_TERMS terms, in order)
//   out[n] = (x[n] - mean) / sqrt(var + eps) * w + b,     var = mean((x - mean)^2)
//
// The stream is 32-bit and all of the arithmetic is; the terms are branch outputs in the
// compute dtype.  Without out_rows every token is normed and the stream is updated in place;
// with out_rows only the listed tokens are normed (out is then [rows, d]) and the stream is not
// written.  out may be the stream itself (32-bit output, no terms: a norm of the stream in
// place, as a model applies to its embedding output).
// One CTA per token; the row waits in shared memory between the three passes (sum, squared
// deviations, output), so a token's result does not depend on its neighbours.
#include "common.cuh"

namespace sllm {

constexpr int LN_MAX_TERMS = 4;
constexpr int LN_THREADS = 256;

struct LnTerms {
    const void* p[LN_MAX_TERMS];
    float coef[LN_MAX_TERMS];
    int n;
};

template <typename TD, typename TO>
__global__ void __launch_bounds__(LN_THREADS)
add_layernorm_kernel(float* resid, const LnTerms terms, const float* __restrict__ w,
                     const float* __restrict__ b, float eps, TO* out,
                     const int* __restrict__ out_rows, int d) {
    extern __shared__ float row[];      // [d]
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int64_t n = out_rows ? out_rows[blockIdx.x] : blockIdx.x;
    float* r = resid + n * d;
    float sum = 0.f;
    for (int c = threadIdx.x; c < d; c += LN_THREADS) {
        float x = r[c];
#pragma unroll
        for (int i = 0; i < LN_MAX_TERMS; ++i)
            if (i < terms.n)
                x = fmaf(terms.coef[i], to_float(reinterpret_cast<const TD*>(terms.p[i])[n * d + c]), x);
        if (terms.n > 0 && out_rows == nullptr) r[c] = x;
        row[c] = x;
        sum += x;
    }
    const float mean = block_sum(sum, scratch) / (float)d;
    float dev = 0.f;
    for (int c = threadIdx.x; c < d; c += LN_THREADS) {
        const float e = row[c] - mean;
        dev = fmaf(e, e, dev);
    }
    const float inv = 1.0f / sqrtf(block_sum(dev, scratch) / (float)d + eps);
    TO* o = out + (int64_t)blockIdx.x * d;
    for (int c = threadIdx.x; c < d; c += LN_THREADS)
        o[c] = from_float<TO>((row[c] - mean) * inv * w[c] + b[c]);
}

// Four elements at a time (d a multiple of 4, every base 16-byte aligned): the same sums in
// another order.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
    return make_float4(__low2float(h[0]), __high2float(h[0]), __low2float(h[1]), __high2float(h[1]));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    uint2 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
    h[0] = __floats2bfloat162_rn(v.x, v.y);
    h[1] = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = r;
}

template <typename TD, typename TO>
__global__ void __launch_bounds__(LN_THREADS)
add_layernorm_vec_kernel(float* resid, const LnTerms terms, const float* __restrict__ w,
                         const float* __restrict__ b, float eps, TO* out,
                         const int* __restrict__ out_rows, int d) {
    extern __shared__ __align__(16) float row[];      // [d]
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int64_t n = out_rows ? out_rows[blockIdx.x] : blockIdx.x;
    float* r = resid + n * d;
    float sum = 0.f;
    for (int c = threadIdx.x * 4; c < d; c += LN_THREADS * 4) {
        float4 x = load4(r + c);
#pragma unroll
        for (int i = 0; i < LN_MAX_TERMS; ++i)
            if (i < terms.n) {
                const float4 t = load4(reinterpret_cast<const TD*>(terms.p[i]) + n * d + c);
                x.x = fmaf(terms.coef[i], t.x, x.x); x.y = fmaf(terms.coef[i], t.y, x.y);
                x.z = fmaf(terms.coef[i], t.z, x.z); x.w = fmaf(terms.coef[i], t.w, x.w);
            }
        if (terms.n > 0 && out_rows == nullptr) store4(r + c, x);
        store4(row + c, x);
        sum += (x.x + x.y) + (x.z + x.w);
    }
    const float mean = block_sum(sum, scratch) / (float)d;
    float dev = 0.f;
    for (int c = threadIdx.x * 4; c < d; c += LN_THREADS * 4) {
        const float4 x = load4(row + c);
        const float e0 = x.x - mean, e1 = x.y - mean, e2 = x.z - mean, e3 = x.w - mean;
        dev += (e0 * e0 + e1 * e1) + (e2 * e2 + e3 * e3);
    }
    const float inv = 1.0f / sqrtf(block_sum(dev, scratch) / (float)d + eps);
    TO* o = out + (int64_t)blockIdx.x * d;
    for (int c = threadIdx.x * 4; c < d; c += LN_THREADS * 4) {
        const float4 x = load4(row + c), g = load4(w + c), h = load4(b + c);
        store4(o + c, make_float4((x.x - mean) * inv * g.x + h.x, (x.y - mean) * inv * g.y + h.y,
                                  (x.z - mean) * inv * g.z + h.z, (x.w - mean) * inv * g.w + h.w));
    }
}

}  // namespace sllm

using namespace sllm;

// resid: float [n_tokens, d].  terms: n_terms pointers to [n_tokens, d] tensors of dtype
// term_dtype (0 = float32, 1 = bfloat16) with their coefficients.  out: [n_out, d] of out_dtype,
// n_out = n_rows if out_rows (int [n_rows]) is given, else n_tokens.
SLLM_EXPORT int sllm_add_layernorm(float* resid, const void* const* term_ptrs,
                                   const float* term_coefs, int n_terms, int term_dtype,
                                   const float* w, const float* b, float eps, void* out,
                                   int out_dtype, const int* out_rows, int n_out, int d,
                                   cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (d <= 0 || d > 32768 || n_terms < 0 || n_terms > LN_MAX_TERMS)
        return (int)cudaErrorInvalidValue;
    LnTerms t;
    t.n = n_terms;
    for (int i = 0; i < LN_MAX_TERMS; ++i) {
        t.p[i] = i < n_terms ? term_ptrs[i] : nullptr;
        t.coef[i] = i < n_terms ? term_coefs[i] : 0.f;
    }
    const size_t smem = (size_t)d * sizeof(float);
    bool vec = d % 4 == 0 && !(((uintptr_t)resid | (uintptr_t)w | (uintptr_t)b | (uintptr_t)out) & 15);
    for (int i = 0; i < n_terms; ++i) vec = vec && !((uintptr_t)term_ptrs[i] & 15);
#define SLLM_LN_LAUNCH(TD, TO)                                                                  \
    do {                                                                                        \
        if (smem > 48 * 1024) {                                                                 \
            cudaError_t e = cudaFuncSetAttribute(add_layernorm_kernel<TD, TO>,                  \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                                 (int)smem);                                    \
            if (e != cudaSuccess) return (int)e;                                                \
        }                                                                                       \
        if (vec && smem <= 48 * 1024) {                                                         \
            cudaError_t e = sllm_launch_pdl(add_layernorm_vec_kernel<TD, TO>, dim3(n_out),      \
                                            dim3(LN_THREADS), smem, stream, resid, t, w, b,     \
                                            eps, (TO*)out, out_rows, d);                        \
            if (e != cudaSuccess) return (int)e;                                                \
            break;                                                                              \
        }                                                                                       \
        cudaError_t e = sllm_launch_pdl(add_layernorm_kernel<TD, TO>, dim3(n_out),              \
                                        dim3(LN_THREADS), smem, stream, resid, t, w, b, eps,    \
                                        (TO*)out, out_rows, d);                                 \
        if (e != cudaSuccess) return (int)e;                                                    \
    } while (0)
    if (term_dtype == 0 && out_dtype == 0) SLLM_LN_LAUNCH(float, float);
    else if (term_dtype == 1 && out_dtype == 1) SLLM_LN_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (term_dtype == 1 && out_dtype == 0) SLLM_LN_LAUNCH(__nv_bfloat16, float);
    else if (term_dtype == 0 && out_dtype == 1) SLLM_LN_LAUNCH(float, __nv_bfloat16);
    else return (int)cudaErrorInvalidValue;
#undef SLLM_LN_LAUNCH
    return 0;
}
