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
#define SLLM_LN_LAUNCH(TD, TO)                                                                  \
    do {                                                                                        \
        if (smem > 48 * 1024) {                                                                 \
            cudaError_t e = cudaFuncSetAttribute(add_layernorm_kernel<TD, TO>,                  \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                                 (int)smem);                                    \
            if (e != cudaSuccess) return (int)e;                                                \
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
