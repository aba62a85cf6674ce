// Elementwise kernels of layers that norm a branch's OUTPUT before it joins the residual
// stream (x <- x + norm(branch(x))), and of what such layers put around their products:
//
//   * embedding gather with a sinusoidal position vector added, and a copy of the stream in
//     the compute dtype for the first branch to read;
//   * resid += rmsnorm(delta) * gain, again with the copy for the next branch;
//   * gated activations act(gate) * up with the activation as a parameter (silu, tanh-gelu);
//   * x *= sigmoid(gate) (an output gate on a mixer's heads);
//   * act(a) * table[token, columns] (a per-token side input gathered from a table).
//
// The residual stream is 32-bit; T is the dtype of matrix-product operands (float in the
// 32-bit path, bfloat16 in the serving path).  Norms, angles and activations are computed in
// 32-bit and rounded once.
#include "common.cuh"

namespace sllm {

__device__ __forceinline__ float act_silu(float z) { return z / (1.0f + expf(-z)); }
// 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
__device__ __forceinline__ float act_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float activate(float z, int act) {
    return act == 1 ? act_gelu_tanh(z) : act_silu(z);
}

// out[n, e] = table[ids[n], e] * scale + pe(positions[n], e), where, with inv_freq != nullptr,
// pe(p, 2i) = sin(p * inv_freq[i]) and pe(p, 2i + 1) = cos(p * inv_freq[i]) (angles in 32-bit),
// else 0.  cast_out (may be null) gets the same row rounded to T.  An id -1 - j stands for
// pending[j].  One block per token.
template <typename T>
__global__ void embed_positional_kernel(const int* __restrict__ ids, const int* __restrict__ pending,
                                        const int* __restrict__ positions,
                                        const T* __restrict__ table, float* __restrict__ out,
                                        T* __restrict__ cast_out, int d, float scale,
                                        const float* __restrict__ inv_freq) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    int id = ids[n];
    if (id < 0) id = pending[-1 - id];
    const float p = (float)positions[n];
    const T* src = table + (int64_t)id * d;
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        float v = to_float(src[e]) * scale;
        if (inv_freq) {
            const float angle = p * inv_freq[e >> 1];
            v += (e & 1) ? cosf(angle) : sinf(angle);
        }
        out[n * d + e] = v;
        if (cast_out) cast_out[n * d + e] = from_float<T>(v);
    }
}

// resid[n] += delta[n] / sqrt(mean(delta[n]^2) + eps) * gain; cast_out[n] (may be null) =
// T(resid[n]).  One block per token; the row of delta stays in registers between the passes
// when it is short enough, else it is read twice.
template <typename T>
__global__ void add_normed_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                  const float* __restrict__ gain, float eps,
                                  T* __restrict__ cast_out, int d,
                                  const float* __restrict__ gain2, float eps2,
                                  T* __restrict__ out2) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[33];
    const int64_t n = blockIdx.x;
    const T* dl = delta + n * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = to_float(dl[i]);
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)d + eps);
    float* x = resid + n * d;
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = x[i] + to_float(dl[i]) * inv * gain[i];
        x[i] = v;
        ss2 += v * v;
        if (cast_out) cast_out[n * d + i] = from_float<T>(v);
    }
    if (!out2) return;
    // the norm in front of the next branch, on the row as it now is (a thread reads back what
    // it has written itself)
    const float inv2 = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)d + eps2);
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        out2[n * d + i] = from_float<T>(x[i] * inv2 * gain2[i]);
}

// add_normed_kernel with 16-byte accesses (d a multiple of Vec<T>::N, rows 16-byte aligned).
// The sum of squares is added up in the order of the scalar kernel's threads only if the block
// sizes agree; the two kernels differ by the order of a 32-bit sum, nothing else.
template <typename T>
__global__ void add_normed_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                      const float* __restrict__ gain, float eps,
                                      T* __restrict__ cast_out, int d,
                                      const float* __restrict__ gain2, float eps2,
                                      T* __restrict__ out2) {
    pdl_wait();
    pdl_trigger();
    constexpr int N = Vec<T>::N;
    __shared__ float scratch[33];
    const int64_t n = blockIdx.x;
    const T* dl = delta + n * d;
    float first[N];
    float ss = 0.f;
    for (int i = threadIdx.x * N; i < d; i += blockDim.x * N) {
        float v[N];
        Vec<T>::load(dl + i, v);
#pragma unroll
        for (int w = 0; w < N; ++w) {
            ss += v[w] * v[w];
            if (i == (int)threadIdx.x * N) first[w] = v[w];   // most rows fit one pass
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)d + eps);
    float* x = resid + n * d;
    float ss2 = 0.f;
    for (int i = threadIdx.x * N; i < d; i += blockDim.x * N) {
        float v[N], y[N];
        if (i == (int)threadIdx.x * N) {
#pragma unroll
            for (int w = 0; w < N; ++w) v[w] = first[w];
        } else {
            Vec<T>::load(dl + i, v);
        }
#pragma unroll
        for (int q = 0; q < N; q += 4) {
            const float4 r = *reinterpret_cast<const float4*>(x + i + q);
            const float4 g = *reinterpret_cast<const float4*>(gain + i + q);
            y[q] = r.x + v[q] * inv * g.x;
            y[q + 1] = r.y + v[q + 1] * inv * g.y;
            y[q + 2] = r.z + v[q + 2] * inv * g.z;
            y[q + 3] = r.w + v[q + 3] * inv * g.w;
            *reinterpret_cast<float4*>(x + i + q) = make_float4(y[q], y[q + 1], y[q + 2], y[q + 3]);
        }
#pragma unroll
        for (int w = 0; w < N; ++w) {
            ss2 += y[w] * y[w];
            if (i == (int)threadIdx.x * N) first[w] = y[w];
        }
        if (cast_out) Vec<T>::store(cast_out + n * d + i, y);
    }
    if (!out2) return;
    // the norm in front of the next branch, on the row as it now is (beyond its first pass a
    // thread reads back what it has written itself)
    const float inv2 = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)d + eps2);
    for (int i = threadIdx.x * N; i < d; i += blockDim.x * N) {
        float y[N];
#pragma unroll
        for (int q = 0; q < N; q += 4) {
            float4 r;
            if (i == (int)threadIdx.x * N) r = make_float4(first[q], first[q + 1], first[q + 2], first[q + 3]);
            else r = *reinterpret_cast<const float4*>(x + i + q);
            const float4 g = *reinterpret_cast<const float4*>(gain2 + i + q);
            y[q] = r.x * inv2 * g.x;
            y[q + 1] = r.y * inv2 * g.y;
            y[q + 2] = r.z * inv2 * g.z;
            y[q + 3] = r.w * inv2 * g.w;
        }
        Vec<T>::store(out2 + n * d + i, y);
    }
}

// out[n, f] = act(gu[n, f]) * gu[n, F + f] in 32-bit.
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t n_rows,
                                 int F, int act) {
    pdl_wait();
    pdl_trigger();
    const int64_t total = n_rows * F;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / F;
        const int f = (int)(i - n * F);
        const float g = to_float(gu[n * 2 * F + f]);
        const float u = to_float(gu[n * 2 * F + F + f]);
        out[i] = from_float<T>(activate(g, act) * u);
    }
}

// A gated feed-forward's activation with clamps: with g = min(gu[n, f], limit) and
// u = clamp(gu[n, F + f], -limit, limit),  out[n, f] = g * sigmoid(slope * g) * (u + 1), in
// 32-bit.  out rows are ldo apart (a column slice of a wider buffer).
template <typename T>
__global__ void clamped_gate_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t ldo,
                                    int64_t n_rows, int F, float limit, float slope) {
    pdl_wait();
    pdl_trigger();
    const int64_t total = n_rows * F;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / F;
        const int f = (int)(i - n * F);
        const float g = fminf(to_float(gu[n * 2 * F + f]), limit);
        const float u = fminf(fmaxf(to_float(gu[n * 2 * F + F + f]), -limit), limit);
        out[n * ldo + f] = from_float<T>(g / (1.0f + expf(-slope * g)) * (u + 1.0f));
    }
}

// x[n, c] *= sigmoid(gate[n, c]) for c < C; x rows ldx apart, gate rows ldg apart.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, int64_t ldx, const T* __restrict__ gate,
                                    int64_t ldg, int64_t n_rows, int C) {
    pdl_wait();
    pdl_trigger();
    const int64_t total = n_rows * C;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / C;
        const int c = (int)(i - n * C);
        const float g = to_float(gate[n * ldg + c]);
        x[n * ldx + c] = from_float<T>(to_float(x[n * ldx + c]) / (1.0f + expf(-g)));
    }
}

// sigmoid_gate_kernel with 16-byte accesses (C, ldx, ldg multiples of Vec<T>::N, 16-byte bases).
template <typename T>
__global__ void sigmoid_gate_vec_kernel(T* __restrict__ x, int64_t ldx, const T* __restrict__ gate,
                                        int64_t ldg, int64_t n_rows, int C) {
    pdl_wait();
    pdl_trigger();
    constexpr int N = Vec<T>::N;
    const int per_row = C / N;
    const int64_t total = n_rows * per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / per_row;
        const int c = (int)(i - n * per_row) * N;
        float v[N], g[N];
        Vec<T>::load(x + n * ldx + c, v);
        Vec<T>::load(gate + n * ldg + c, g);
#pragma unroll
        for (int w = 0; w < N; ++w) v[w] = v[w] / (1.0f + expf(-g[w]));
        Vec<T>::store(x + n * ldx + c, v);
    }
}

// out[n, j] = act(a[n, j]) * table[ids[n], col0 + j] for j < dim; table rows ld_table apart.
template <typename T>
__global__ void side_gate_kernel(const T* __restrict__ a, const int* __restrict__ ids,
                                 const int* __restrict__ pending, const T* __restrict__ table,
                                 int64_t ld_table, int col0, int dim, int act,
                                 T* __restrict__ out, int64_t n_rows) {
    pdl_wait();
    pdl_trigger();
    const int64_t total = n_rows * dim;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / dim;
        const int j = (int)(i - n * dim);
        int id = ids[n];
        if (id < 0) id = pending[-1 - id];
        const float e = to_float(table[(int64_t)id * ld_table + col0 + j]);
        out[i] = from_float<T>(activate(to_float(a[i]), act) * e);
    }
}

// An activation with two numbers of its own, element by element: out = act(x; p0, p1).
//   act 0 (xIELU with its two factors ready): x > 0: p0 x^2 + x / 2;
//                                             x <= 0: p1 (exp(x) - 1 - x) + x / 2.
template <bool FAST>
__device__ __forceinline__ float param_activate(float z, int act, float p0, float p1) {
    (void)act;
    // FAST (results that are rounded to bfloat16): exp(z) - 1 with the hardware's exponential,
    // whose absolute error of 1e-7 is far below that rounding wherever the term matters
    const float em1 = FAST ? __expf(z) - 1.0f : expm1f(z);
    return z > 0.f ? fmaf(p0 * z, z, 0.5f * z) : fmaf(p1, em1 - z, 0.5f * z);
}
template <typename T> struct RoundsToBf16 { static constexpr bool value = false; };
template <> struct RoundsToBf16<__nv_bfloat16> { static constexpr bool value = true; };

template <typename T>
__global__ void param_act_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n, int act,
                                 float p0, float p1) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        out[i] = from_float<T>(param_activate<RoundsToBf16<T>::value>(to_float(x[i]), act, p0, p1));
}

template <typename T>
__global__ void param_act_vec_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n_units,
                                     int act, float p0, float p1) {
    pdl_wait();
    pdl_trigger();
    constexpr int N = Vec<T>::N;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_units;
         i += (int64_t)gridDim.x * blockDim.x) {
        float v[N];
        Vec<T>::load(x + i * N, v);
#pragma unroll
        for (int w = 0; w < N; ++w) v[w] = param_activate<RoundsToBf16<T>::value>(v[w], act, p0, p1);
        Vec<T>::store(out + i * N, v);
    }
}

// out[n] = [a[n]; b[n]] rounded to T: two 32-bit streams side by side, as the operand of a
// product over both.
template <typename T>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                   T* __restrict__ out, int64_t total, int d) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / (2 * d);
        const int e = (int)(i - n * 2 * d);
        out[i] = from_float<T>(e < d ? a[n * d + e] : b[n * d + e - d]);
    }
}

// concat_cast_kernel for d a multiple of 8 and 16-byte aligned rows: a thread takes 8
// neighbouring entries of one of the two streams (two 16-byte loads) and stores them at once.
template <typename T>
__global__ void concat_cast_vec_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                       T* __restrict__ out, int64_t total8, int d) {
    pdl_wait();
    pdl_trigger();
    const int per_row = 2 * d / 8;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total8;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / per_row;
        const int e = (int)(i - n * per_row) * 8;
        const float* src = e < d ? a + n * d + e : b + n * d + (e - d);
        const float4 lo = *reinterpret_cast<const float4*>(src);
        const float4 hi = *reinterpret_cast<const float4*>(src + 4);
        T* dst = out + n * 2 * d + e;
        if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(dst) = lo;
            *reinterpret_cast<float4*>(dst + 4) = hi;
        } else {
            const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            Vec<T>::store(dst, v);
        }
    }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_concat_cast(const float* a, const float* b, void* out, int n_rows, int d,
                                 int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) return (int)cudaErrorInvalidValue;
    const int64_t total = (int64_t)n_rows * 2 * d;
    if (d % 8 == 0 && !(((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) && dtype >= 0 &&
        dtype <= 1) {
        const int64_t total8 = total / 8;
        const int vblocks = (int)((total8 + 255) / 256 > 148 * 16 ? 148 * 16 : (total8 + 255) / 256);
        if (dtype == 0)
            return (int)sllm_launch_pdl(concat_cast_vec_kernel<float>, dim3(vblocks), dim3(256), 0,
                                        stream, a, b, (float*)out, total8, d);
        return (int)sllm_launch_pdl(concat_cast_vec_kernel<__nv_bfloat16>, dim3(vblocks), dim3(256),
                                    0, stream, a, b, (__nv_bfloat16*)out, total8, d);
    }
    const int blocks = (int)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256);
    if (dtype == 0)
        return (int)sllm_launch_pdl(concat_cast_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                                    a, b, (float*)out, total, d);
    if (dtype == 1)
        return (int)sllm_launch_pdl(concat_cast_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0,
                                    stream, a, b, (__nv_bfloat16*)out, total, d);
    return (int)cudaErrorInvalidValue;
}

static int row_threads(int d) {
    int t = 32;
    while (t < 1024 && t * 4 < d) t <<= 1;
    return t;
}

static int flat_blocks(int64_t total, int threads) {
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    return (int)blocks;
}

#define SLLM_BY_DTYPE(dtype, CALL_F32, CALL_BF16)         \
    do {                                                  \
        if ((dtype) == 0) { CALL_F32; }                   \
        else if ((dtype) == 1) { CALL_BF16; }             \
        else return (int)cudaErrorInvalidValue;           \
        SLLM_LAUNCH_CHECK();                              \
    } while (0)

// dtype: 0 = float32, 1 = bfloat16 (of table / delta / cast_out / gu / x / a).
SLLM_EXPORT int sllm_embed_positional(const int* ids, const int* pending, const int* positions,
                                      const void* table, float* out, void* cast_out, int n_tokens,
                                      int d, int dtype, float scale, const float* inv_freq,
                                      cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0) return (int)cudaErrorInvalidValue;
    const int threads = row_threads(d);
    SLLM_BY_DTYPE(dtype,
        (embed_positional_kernel<float><<<n_tokens, threads, 0, stream>>>(
            ids, pending, positions, (const float*)table, out, (float*)cast_out, d, scale, inv_freq)),
        (embed_positional_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            ids, pending, positions, (const __nv_bfloat16*)table, out, (__nv_bfloat16*)cast_out, d,
            scale, inv_freq)));
    return 0;
}

// gain2 / eps2 / out2 (or nulls): out2 = T(rmsnorm(resid as updated) * gain2), the norm in front of
// the next branch, from the same pass.
SLLM_EXPORT int sllm_add_normed(float* resid, const void* delta, const float* gain, float eps,
                                void* cast_out, const float* gain2, float eps2, void* out2,
                                int n_tokens, int d, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || (out2 && !gain2)) return (int)cudaErrorInvalidValue;
    const int vec = dtype == 0 ? 4 : 8;
    const bool aligned = !(((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)gain |
                            (uintptr_t)cast_out | (uintptr_t)gain2 | (uintptr_t)out2) & 15);
    if (d % vec == 0 && aligned && dtype >= 0 && dtype <= 1) {
        int vt = 32;
        while (vt < 512 && vt * vec < d) vt <<= 1;
        SLLM_BY_DTYPE(dtype,
            (add_normed_vec_kernel<float><<<n_tokens, vt, 0, stream>>>(
                resid, (const float*)delta, gain, eps, (float*)cast_out, d, gain2, eps2,
                (float*)out2)),
            (add_normed_vec_kernel<__nv_bfloat16><<<n_tokens, vt, 0, stream>>>(
                resid, (const __nv_bfloat16*)delta, gain, eps, (__nv_bfloat16*)cast_out, d, gain2,
                eps2, (__nv_bfloat16*)out2)));
        return 0;
    }
    const int threads = row_threads(d);
    SLLM_BY_DTYPE(dtype,
        (add_normed_kernel<float><<<n_tokens, threads, 0, stream>>>(
            resid, (const float*)delta, gain, eps, (float*)cast_out, d, gain2, eps2,
            (float*)out2)),
        (add_normed_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            resid, (const __nv_bfloat16*)delta, gain, eps, (__nv_bfloat16*)cast_out, d, gain2,
            eps2, (__nv_bfloat16*)out2)));
    return 0;
}

// act: 0 = silu, 1 = gelu (tanh form).
SLLM_EXPORT int sllm_gated_act(const void* gu, void* out, int n_rows, int F, int act, int dtype,
                               cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (F <= 0 || act < 0 || act > 1) return (int)cudaErrorInvalidValue;
    const int blocks = flat_blocks((int64_t)n_rows * F, 256);
    SLLM_BY_DTYPE(dtype,
        (gated_act_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, (float*)out, n_rows,
                                                             F, act)),
        (gated_act_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
            (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_rows, F, act)));
    return 0;
}

SLLM_EXPORT int sllm_clamped_gate(const void* gu, void* out, int64_t ldo, int n_rows, int F,
                                  float limit, float slope, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (F <= 0 || ldo < F || !(limit > 0.f)) return (int)cudaErrorInvalidValue;
    const int blocks = flat_blocks((int64_t)n_rows * F, 256);
    SLLM_BY_DTYPE(dtype,
        (clamped_gate_kernel<float><<<blocks, 256, 0, stream>>>(
            (const float*)gu, (float*)out, ldo, n_rows, F, limit, slope)),
        (clamped_gate_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
            (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, ldo, n_rows, F, limit, slope)));
    return 0;
}

SLLM_EXPORT int sllm_sigmoid_gate(void* x, int64_t ldx, const void* gate, int64_t ldg, int n_rows,
                                  int C, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (C <= 0) return (int)cudaErrorInvalidValue;
    const int vec = dtype == 0 ? 4 : 8;
    if (C % vec == 0 && ldx % vec == 0 && ldg % vec == 0 &&
        !(((uintptr_t)x | (uintptr_t)gate) & 15) && dtype >= 0 && dtype <= 1) {
        const int vblocks = flat_blocks((int64_t)n_rows * (C / vec), 256);
        SLLM_BY_DTYPE(dtype,
            (sigmoid_gate_vec_kernel<float><<<vblocks, 256, 0, stream>>>(
                (float*)x, ldx, (const float*)gate, ldg, n_rows, C)),
            (sigmoid_gate_vec_kernel<__nv_bfloat16><<<vblocks, 256, 0, stream>>>(
                (__nv_bfloat16*)x, ldx, (const __nv_bfloat16*)gate, ldg, n_rows, C)));
        return 0;
    }
    const int blocks = flat_blocks((int64_t)n_rows * C, 256);
    SLLM_BY_DTYPE(dtype,
        (sigmoid_gate_kernel<float><<<blocks, 256, 0, stream>>>((float*)x, ldx, (const float*)gate,
                                                                ldg, n_rows, C)),
        (sigmoid_gate_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
            (__nv_bfloat16*)x, ldx, (const __nv_bfloat16*)gate, ldg, n_rows, C)));
    return 0;
}

SLLM_EXPORT int sllm_side_gate(const void* a, const int* ids, const int* pending, const void* table,
                               int64_t ld_table, int col0, int dim, int act, void* out, int n_rows,
                               int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (dim <= 0 || col0 < 0 || act < 0 || act > 1) return (int)cudaErrorInvalidValue;
    const int blocks = flat_blocks((int64_t)n_rows * dim, 128);
    SLLM_BY_DTYPE(dtype,
        (side_gate_kernel<float><<<blocks, 128, 0, stream>>>(
            (const float*)a, ids, pending, (const float*)table, ld_table, col0, dim, act,
            (float*)out, n_rows)),
        (side_gate_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(
            (const __nv_bfloat16*)a, ids, pending, (const __nv_bfloat16*)table, ld_table, col0, dim,
            act, (__nv_bfloat16*)out, n_rows)));
    return 0;
}

// act: 0 = xIELU (p0 the factor of x^2 for x > 0, p1 the factor of exp(x) - 1 - x for x <= 0).
SLLM_EXPORT int sllm_param_act(const void* x, void* out, int64_t n, int act, float p0, float p1,
                               int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (act != 0 || dtype < 0 || dtype > 1) return (int)cudaErrorInvalidValue;
    const int vec = dtype == 0 ? 4 : 8;
    if (n % vec == 0 && !(((uintptr_t)x | (uintptr_t)out) & 15)) {
        const int64_t units = n / vec;
        int64_t blocks = (units + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        SLLM_BY_DTYPE(dtype,
            (param_act_vec_kernel<float><<<(int)blocks, 256, 0, stream>>>(
                (const float*)x, (float*)out, units, act, p0, p1)),
            (param_act_vec_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
                (const __nv_bfloat16*)x, (__nv_bfloat16*)out, units, act, p0, p1)));
        return 0;
    }
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    SLLM_BY_DTYPE(dtype,
        (param_act_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)x, (float*)out, n,
                                                                  act, p0, p1)),
        (param_act_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
            (const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, act, p0, p1)));
    return 0;
}
