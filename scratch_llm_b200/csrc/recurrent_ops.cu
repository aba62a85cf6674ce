// What stands around a linear recurrence in a recurrent mixer: the short causal convolution
// over time with its carried inputs, and the per-head norm and gate of the read-out.
//
//   conv:   y[t, c] = silu( sum_j taps[c, j] * x[t - (K - 1 - j), c] ),  j = 0 .. K-1
//           (the last tap multiplies the current token; before a sequence's start x is 0).
//           A request's last K - 1 inputs are carried in its state slot, state[slot, s, c] with
//           s = K - 2 the most recent, so that a row may bring any number of tokens per step.
//   update: the state after the row's tokens (a launch of its own: the convolution of a row's
//           first tokens reads the old state while its last tokens would overwrite it).
//   read-out: out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * gain * silu(gate[t, h, :])
//
// T is the dtype of matrix-product operands (float / bfloat16); taps, gains and the read-out
// o are 32-bit.  Tokens whose row is -1 are padding: their outputs are zero, nothing is carried.
#include "common.cuh"

namespace sllm {

constexpr int CONV_MAX_TAPS = 16;

// x: [n_tokens, ldx], the convolved channels are its first C columns.  out: [n_tokens, C].
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ x, int64_t ldx,
                                 const float* __restrict__ taps, int K,
                                 const T* __restrict__ state, const int* __restrict__ token_row,
                                 const int* __restrict__ row_start,
                                 const int* __restrict__ row_slot, T* __restrict__ out, int C,
                                 int64_t n_tokens) {
    pdl_wait();
    pdl_trigger();
    const int64_t total = n_tokens * C;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = idx / C;
        const int c = (int)(idx - n * C);
        const int r = token_row[n];
        if (r < 0) {
            out[idx] = from_float<T>(0.f);
            continue;
        }
        const int i = (int)(n - row_start[r]);           // index of the token within its row
        const T* st = state + (int64_t)row_slot[r] * (K - 1) * C;
        float acc = 0.f;
        for (int j = 0; j < K; ++j) {
            const int back = K - 1 - j;                  // how many tokens before this one
            float v;
            if (back <= i) v = to_float(x[(n - back) * ldx + c]);
            else v = to_float(st[(int64_t)(i + j) * C + c]);   // i - back + (K - 1)
            acc = fmaf(taps[(int64_t)c * K + j], v, acc);
        }
        out[idx] = from_float<T>(acc / (1.0f + expf(-acc)));
    }
}

// The same for bfloat16 with 16-byte accesses: a thread takes 8 consecutive channels of a token
// (C, ldx multiples of 8; 16-byte bases).  The arithmetic and its order are the scalar kernel's.
// taps_t is the taps' transpose [K, C], so that a thread's 8 taps of one time step are 32
// consecutive bytes and a warp's are consecutive too.
__global__ void conv_silu_vec_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                     const float* __restrict__ taps_t, int K,
                                     const __nv_bfloat16* __restrict__ state,
                                     const int* __restrict__ token_row,
                                     const int* __restrict__ row_start,
                                     const int* __restrict__ row_slot,
                                     __nv_bfloat16* __restrict__ out, int C, int64_t n_tokens) {
    pdl_wait();
    pdl_trigger();
    typedef __nv_bfloat16 bf16;
    const int per_row = C / 8;
    const int64_t total = n_tokens * per_row;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = idx / per_row;
        const int c = (int)(idx - n * per_row) * 8;
        const int r = token_row[n];
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);
        if (r >= 0) {
            const int i = (int)(n - row_start[r]);
            const bf16* st = state + (int64_t)row_slot[r] * (K - 1) * C;
            float acc[8];
#pragma unroll
            for (int w = 0; w < 8; ++w) acc[w] = 0.f;
            for (int j = 0; j < K; ++j) {
                const int back = K - 1 - j;
                const bf16* src = back <= i ? x + (n - back) * ldx + c : st + (int64_t)(i + j) * C + c;
                const uint4 raw = *reinterpret_cast<const uint4*>(src);
                const bf16* e = reinterpret_cast<const bf16*>(&raw);
                const float4 ta = *reinterpret_cast<const float4*>(taps_t + (int64_t)j * C + c);
                const float4 tb = *reinterpret_cast<const float4*>(taps_t + (int64_t)j * C + c + 4);
                const float tp[8] = {ta.x, ta.y, ta.z, ta.w, tb.x, tb.y, tb.z, tb.w};
#pragma unroll
                for (int w = 0; w < 8; ++w) acc[w] = fmaf(tp[w], __bfloat162float(e[w]), acc[w]);
            }
            bf16* o = reinterpret_cast<bf16*>(&packed);
#pragma unroll
            for (int w = 0; w < 8; ++w) o[w] = __float2bfloat16_rn(acc[w] / (1.0f + expf(-acc[w])));
        }
        *reinterpret_cast<uint4*>(out + n * C + c) = packed;
    }
}

// state[slot, s, c] for s = 0 .. K-2 becomes entry n_new + s of (old state, the row's new inputs).
// grid (ceil(C / 256), rows); rows without tokens are left alone.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, int64_t ldx, int K,
                                         T* __restrict__ state, const int* __restrict__ row_start,
                                         const int* __restrict__ row_slot, int C) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t0 = row_start[r], n_new = row_start[r + 1] - t0;
    if (c >= C || n_new <= 0) return;
    T* st = state + (int64_t)row_slot[r] * (K - 1) * C;
    // ascending s reads old entries n_new + s > s only: in place is safe
    for (int s = 0; s < K - 1; ++s) {
        const int src = n_new + s;
        st[(int64_t)s * C + c] = src < K - 1 ? st[(int64_t)src * C + c]
                                             : x[(int64_t)(t0 + src - (K - 1)) * ldx + c];
    }
}

// grid (tokens, ceil(H / 4)); one warp per (token, head).  o: [n_tokens, H * V] float;
// gate: rows ldg apart; out: rows ldo apart (a column slice of a wider buffer, or H * V).  gain has V entries (every head the same) or,
// with gain_per_head, H * V.  gate_act: 0 = silu(gate), 1 = sigmoid(gate).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int64_t ldg,
                      const float* __restrict__ gain, float eps, T* __restrict__ out, int64_t ldo,
                      int H, int V, int gain_per_head, int gate_act) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    const int head = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head >= H) return;
    const float* src = o + (n * H + head) * V;
    float ss = 0.f;
    for (int j = lane; j < V; j += 32) ss += src[j] * src[j];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)V + eps);
    const T* g = gate + n * ldg + (int64_t)head * V;
    const float* gn = gain + (gain_per_head ? (int64_t)head * V : 0);
    T* dst = out + n * ldo + (int64_t)head * V;
    for (int j = lane; j < V; j += 32) {
        const float z = to_float(g[j]);
        const float sig = 1.0f / (1.0f + expf(-z));
        dst[j] = from_float<T>(src[j] * inv * gn[j] * (gate_act == 1 ? sig : z * sig));
    }
}

// Decays and removal rates of a delta-rule mixer whose decay comes through a low-rank pair of
// matrices.  pre: float32 [N, ldp] holds the removal rates' inputs in columns [0, C) and the
// low-rank hidden values in columns [C, C + R).  w2t: float32 [R, C] (the second matrix,
// transposed).  out: float32 [N, 2 C]:
//     out[n, c]     = exp(-decay_scale * sigmoid(w0[c] + sum_r w2t[r, c] * tanh(pre[n, C + r])))
//     out[n, C + c] = sigmoid(pre[n, c] + a_bias[c])
// All in 32-bit; the sum runs over r in ascending order for every token, whatever the batch.
// grid (ceil(C / 256), ceil(N / LOWRANK_TOKENS)); shared: LOWRANK_TOKENS * R floats.
constexpr int LOWRANK_TOKENS = 8;
__global__ void __launch_bounds__(256)
lowrank_decay_kernel(const float* __restrict__ pre, int64_t ldp, const float* __restrict__ w2t,
                     const float* __restrict__ w0, const float* __restrict__ a_bias,
                     float decay_scale, float* __restrict__ out, int N, int C, int R) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float th[];   // [LOWRANK_TOKENS][R]
    const int n0 = blockIdx.y * LOWRANK_TOKENS;
    const int nt = min(LOWRANK_TOKENS, N - n0);
    for (int i = threadIdx.x; i < LOWRANK_TOKENS * R; i += blockDim.x) {
        const int t = i / R, r = i - t * R;
        th[t * R + r] = t < nt ? tanhf(pre[(int64_t)(n0 + t) * ldp + C + r]) : 0.f;
    }
    __syncthreads();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float acc[LOWRANK_TOKENS];
#pragma unroll
    for (int t = 0; t < LOWRANK_TOKENS; ++t) acc[t] = 0.f;
    // (sixteen weights are requested at a time: the loop is bound by their latency, not by its
    // arithmetic; tokens beyond nt have zeros in shared memory)
    int r = 0;
    for (; r + 16 <= R; r += 16) {
        float w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = w2t[(int64_t)(r + j) * C + c];
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
            for (int t = 0; t < LOWRANK_TOKENS; ++t) acc[t] = fmaf(w[j], th[t * R + r + j], acc[t]);
    }
    for (; r < R; ++r) {
        const float w = w2t[(int64_t)r * C + c];
#pragma unroll
        for (int t = 0; t < LOWRANK_TOKENS; ++t) acc[t] = fmaf(w, th[t * R + r], acc[t]);
    }
    const float b0 = w0[c], ab = a_bias[c];
#pragma unroll
    for (int t = 0; t < LOWRANK_TOKENS; ++t) {
        if (t < nt) {
            const int64_t n = n0 + t;
            const float sg = 1.0f / (1.0f + expf(-(acc[t] + b0)));
            out[n * 2 * C + c] = expf(-decay_scale * sg);
            out[n * 2 * C + C + c] = 1.0f / (1.0f + expf(-(pre[n * ldp + c] + ab)));
        }
    }
}

// The second product of a low-rank pair, in 32-bit, with what follows it.  pre: float32 [N, ldp]
// holds the hidden values (the first product's output) in columns [col0, col0 + R); w2t: float32
// [R, C] (the second matrix, transposed); bias (may be null): float32 [C].
//     z[n, c] = bias[c] + sum_r w2t[r, c] * pre[n, col0 + r]
//     mode 0:  out = z
//     mode 1:  out = -exp(rate_log[c / per_rate]) * softplus(z)    (the logarithm of a decay
//              exp(-exp(A) softplus(z)) with one A per `per_rate` channels)
// The sum runs over r in ascending order for every token, whatever the batch.  out: [N, C],
// float32 or bfloat16.  One launch serves up to two such products of the same `pre` (a mixer's
// decays and its gate): the first `blocks0` CTAs along x take the first job, the rest the second.
// grid (blocks of both jobs, ceil(N / LOWRANK_TOKENS)); shared: LOWRANK_TOKENS * max R floats.
struct ExpandJob {
    int col0; const float* w2t; const float* bias; const float* rate_log; int per_rate; int mode;
    void* out; int out_bf16; int C; int R;
};

__global__ void __launch_bounds__(256)
lowrank_expand_kernel(const float* __restrict__ pre, int64_t ldp, const ExpandJob j0,
                      const ExpandJob j1, int blocks0, int N) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float th[];   // [LOWRANK_TOKENS][R]
    const bool second = (int)blockIdx.x >= blocks0;
    const ExpandJob& j = second ? j1 : j0;
    const int R = j.R, C = j.C;
    const int n0 = blockIdx.y * LOWRANK_TOKENS;
    const int nt = min(LOWRANK_TOKENS, N - n0);
    for (int i = threadIdx.x; i < LOWRANK_TOKENS * R; i += blockDim.x) {
        const int t = i / R, r = i - t * R;
        th[t * R + r] = t < nt ? pre[(int64_t)(n0 + t) * ldp + j.col0 + r] : 0.f;
    }
    __syncthreads();
    const int c = ((int)blockIdx.x - (second ? blocks0 : 0)) * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float acc[LOWRANK_TOKENS];
#pragma unroll
    for (int t = 0; t < LOWRANK_TOKENS; ++t) acc[t] = 0.f;
    int r = 0;
    for (; r + 16 <= R; r += 16) {
        float w[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) w[k] = j.w2t[(int64_t)(r + k) * C + c];
#pragma unroll
        for (int k = 0; k < 16; ++k)
#pragma unroll
            for (int t = 0; t < LOWRANK_TOKENS; ++t) acc[t] = fmaf(w[k], th[t * R + r + k], acc[t]);
    }
    for (; r < R; ++r) {
        const float w = j.w2t[(int64_t)r * C + c];
#pragma unroll
        for (int t = 0; t < LOWRANK_TOKENS; ++t) acc[t] = fmaf(w, th[t * R + r], acc[t]);
    }
    const float b0 = j.bias ? j.bias[c] : 0.f;
    const float rate = j.mode == 1 ? expf(j.rate_log[c / j.per_rate]) : 0.f;
#pragma unroll
    for (int t = 0; t < LOWRANK_TOKENS; ++t) {
        if (t < nt) {
            float z = acc[t] + b0;
            if (j.mode == 1) z = -rate * (z > 20.f ? z : log1pf(expf(z)));
            const int64_t at = (int64_t)(n0 + t) * C + c;
            if (j.out_bf16) reinterpret_cast<__nv_bfloat16*>(j.out)[at] = __float2bfloat16_rn(z);
            else reinterpret_cast<float*>(j.out)[at] = z;
        }
    }
}

}  // namespace sllm

using namespace sllm;

// dtype: 0 = float32, 1 = bfloat16 (of x, state, out, gate).
// taps_t (may be null): the transpose [K, C] of taps, which the kernel with 16-byte accesses reads.
SLLM_EXPORT int sllm_conv_silu(const void* x, int64_t ldx, const float* taps,
                               const float* taps_t, int K,
                               const void* state, const int* token_row, const int* row_start,
                               const int* row_slot, void* out, int C, int n_tokens, int dtype,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (C <= 0 || K < 1 || K > CONV_MAX_TAPS || ldx < C) return (int)cudaErrorInvalidValue;
    if (dtype == 1 && taps_t != nullptr && C % 8 == 0 && ldx % 8 == 0 &&
        !(((uintptr_t)x | (uintptr_t)state | (uintptr_t)out | (uintptr_t)taps_t) & 15)) {
        int64_t vblocks = ((int64_t)n_tokens * (C / 8) + 255) / 256;
        if (vblocks > 148 * 32) vblocks = 148 * 32;
        conv_silu_vec_kernel<<<(int)vblocks, 256, 0, stream>>>(
            (const __nv_bfloat16*)x, ldx, taps_t, K, (const __nv_bfloat16*)state, token_row,
            row_start, row_slot, (__nv_bfloat16*)out, C, n_tokens);
        SLLM_LAUNCH_CHECK();
        return 0;
    }
    int64_t blocks = ((int64_t)n_tokens * C + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == 0)
        conv_silu_kernel<float><<<(int)blocks, 256, 0, stream>>>(
            (const float*)x, ldx, taps, K, (const float*)state, token_row, row_start, row_slot,
            (float*)out, C, n_tokens);
    else if (dtype == 1)
        conv_silu_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
            (const __nv_bfloat16*)x, ldx, taps, K, (const __nv_bfloat16*)state, token_row,
            row_start, row_slot, (__nv_bfloat16*)out, C, n_tokens);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}

SLLM_EXPORT int sllm_conv_state_update(const void* x, int64_t ldx, int K, void* state,
                                       const int* row_start, const int* row_slot, int C,
                                       int n_rows, int dtype, cudaStream_t stream) {
    if (n_rows <= 0 || K <= 1) return 0;
    if (C <= 0 || K > CONV_MAX_TAPS || n_rows > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((C + 255) / 256, n_rows);
    if (dtype == 0)
        conv_state_update_kernel<float><<<grid, 256, 0, stream>>>(
            (const float*)x, ldx, K, (float*)state, row_start, row_slot, C);
    else if (dtype == 1)
        conv_state_update_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
            (const __nv_bfloat16*)x, ldx, K, (__nv_bfloat16*)state, row_start, row_slot, C);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}

SLLM_EXPORT int sllm_head_norm_gate(const float* o, const void* gate, int64_t ldg,
                                    const float* gain, float eps, void* out, int64_t ldo,
                                    int n_tokens, int H, int V, int gain_per_head, int gate_act,
                                    int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || V <= 0 || gate_act < 0 || gate_act > 1 || ldo < (int64_t)H * V)
        return (int)cudaErrorInvalidValue;
    dim3 grid(n_tokens, (H + 3) / 4);
    if (dtype == 0)
        head_norm_gate_kernel<float><<<grid, 128, 0, stream>>>(o, (const float*)gate, ldg, gain,
                                                               eps, (float*)out, ldo, H, V,
                                                               gain_per_head, gate_act);
    else if (dtype == 1)
        head_norm_gate_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
            o, (const __nv_bfloat16*)gate, ldg, gain, eps, (__nv_bfloat16*)out, ldo, H, V,
            gain_per_head, gate_act);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}

SLLM_EXPORT int sllm_lowrank_decay(const float* pre, int64_t ldp, const float* w2t,
                                   const float* w0, const float* a_bias, float decay_scale,
                                   float* out, int n_tokens, int C, int R, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (C <= 0 || R <= 0 || R > 1024 || ldp < C + R) return (int)cudaErrorInvalidValue;
    dim3 grid((C + 255) / 256, (n_tokens + LOWRANK_TOKENS - 1) / LOWRANK_TOKENS);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    lowrank_decay_kernel<<<grid, 256, LOWRANK_TOKENS * R * sizeof(float), stream>>>(
        pre, ldp, w2t, w0, a_bias, decay_scale, out, n_tokens, C, R);
    SLLM_LAUNCH_CHECK();
    return 0;
}

// Up to two products of one `pre` in a launch (n_jobs 1 or 2); per job: col0, w2t [R, C], bias
// (may be null), rate_log with per_rate (mode 1), mode, out [N, C], out_dtype (0 = float32,
// 1 = bfloat16), C, R.
SLLM_EXPORT int sllm_lowrank_expand(const float* pre, int64_t ldp, int n_jobs, const int* col0,
                                    const float* const* w2t, const float* const* bias,
                                    const float* const* rate_log, const int* per_rate,
                                    const int* mode, void* const* out, const int* out_dtype,
                                    const int* C, const int* R, int n_tokens,
                                    cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_jobs < 1 || n_jobs > 2) return (int)cudaErrorInvalidValue;
    ExpandJob j[2] = {};
    int max_r = 0, max_c = 0;
    for (int i = 0; i < n_jobs; ++i) {
        if (C[i] <= 0 || R[i] <= 0 || R[i] > 1024 || col0[i] < 0 || ldp < col0[i] + R[i] ||
            mode[i] < 0 || mode[i] > 1 || out_dtype[i] < 0 || out_dtype[i] > 1 ||
            (mode[i] == 1 && (!rate_log[i] || per_rate[i] <= 0 || C[i] % per_rate[i])))
            return (int)cudaErrorInvalidValue;
        j[i].col0 = col0[i]; j[i].w2t = w2t[i]; j[i].bias = bias[i]; j[i].rate_log = rate_log[i];
        j[i].per_rate = per_rate[i]; j[i].mode = mode[i]; j[i].out = out[i];
        j[i].out_bf16 = out_dtype[i]; j[i].C = C[i]; j[i].R = R[i];
        max_r = R[i] > max_r ? R[i] : max_r;
        max_c = C[i] > max_c ? C[i] : max_c;
    }
    // steps of few tokens: narrow CTAs, so that the channels spread over more SMs
    const int threads = n_tokens <= 2 * LOWRANK_TOKENS && max_c >= 1024 ? 64 : 256;
    const int blocks0 = (j[0].C + threads - 1) / threads;
    const int blocks1 = n_jobs > 1 ? (j[1].C + threads - 1) / threads : 0;
    dim3 grid(blocks0 + blocks1, (n_tokens + LOWRANK_TOKENS - 1) / LOWRANK_TOKENS);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    lowrank_expand_kernel<<<grid, threads, LOWRANK_TOKENS * max_r * sizeof(float), stream>>>(
        pre, ldp, j[0], j[1], blocks0, n_tokens);
    SLLM_LAUNCH_CHECK();
    return 0;
}
