// Kernels around an attention whose cache holds ONE latent vector per token instead of keys
// and values per head (latent attention in its absorbed form):
//
//   cache[token] = [ rmsnorm(c) * gain  (R entries) | rotated shared key part (r) | zeros ]
//   query[token, head] = [ W_uk_h^T q_unrotated  (R) | rotated q part (r) | zeros ] * 1
//   score = query . cache (times the scale, in the attention kernel); the softmax-weighted sum of
//   the cache vectors' leading R entries is the latent read-out, which W_uv_h turns into the
//   head's output.
//
// The attention itself is the engine's paged kernels with one kv head and one plane per page.
// Here:
//   latent_prep     per token: RMS norm of the query latent (-> cq), RMS norm of the key/value
//                   latent, rotation of the shared key part, store of both into the page
//   latent_q_rot    per (token, head): rotation of the query's rotated part into its place
//                   behind the absorbed part, zeros into the padding
//   head_product    out[n, h, j] = sum_k x[n, h, k] * w[h, j, k] (a product per head; the
//                   32-bit path's absorb and value products, one fixed-order chain per output)
//   head_gate       x[n, h, :] *= sigmoid(gate[n, h])   (one gate per head)
//   latent_small    steps of few tokens: a product per head with the output index last in the
//                   matrix, with the rotated tail (the absorb product and latent_q_rot in one
//                   launch) or with the gate (the value product and head_gate in one launch)
//
// The rotation pairs entry i with entry i + dims / 2 among the first `dims` entries of the rotated
// part: (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * frequency_i, from 32-bit
// tables [positions, dims / 2].  All arithmetic is 32-bit; T is the dtype of the products'
// operands and of the cache.
#include "common.cuh"

namespace sllm {

// a: [N, lda] with the query latent at column 0 (Rq entries) and the key/value latent at column
// kv_col (R entries) followed by the shared key part (r entries).  Two blocks per token: grid
// (N, 2), one for the query latent and one for what is stored.
template <typename T>
__global__ void __launch_bounds__(256)
latent_prep_kernel(const T* __restrict__ a, int64_t lda, int Rq, int kv_col, int R, int r,
                   const float* __restrict__ q_gain, const float* __restrict__ kv_gain, float eps,
                   const int* __restrict__ positions, const int* __restrict__ token_row,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
                   T* __restrict__ cq, T* __restrict__ pages, const int* __restrict__ block_table,
                   int table_stride, int page_size, int Dp, int write, int vec) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[33];
    const int64_t n = blockIdx.x;
    const T* row = a + n * lda;
    float ss = 0.f;
    if (blockIdx.y == 0 && vec) {      // the query latent with 16-byte accesses
        constexpr int VN = Vec<T>::N;
        float first[VN];               // a thread's first vector stays in registers
        for (int e = threadIdx.x * VN; e < Rq; e += blockDim.x * VN) {
            float v[VN];
            Vec<T>::load(row + e, v);
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                ss = fmaf(v[k], v[k], ss);
                if (e == (int)threadIdx.x * VN) first[k] = v[k];
            }
        }
        ss = block_sum(ss, scratch);
        const float q_inv = 1.0f / sqrtf(ss / (float)Rq + eps);
        for (int e = threadIdx.x * VN; e < Rq; e += blockDim.x * VN) {
            float v[VN];
            if (e == (int)threadIdx.x * VN) {
#pragma unroll
                for (int k = 0; k < VN; ++k) v[k] = first[k];
            } else {
                Vec<T>::load(row + e, v);
            }
#pragma unroll
            for (int k = 0; k < VN; k += 4) {
                const float4 g = *reinterpret_cast<const float4*>(q_gain + e + k);
                v[k] *= q_inv * g.x;
                v[k + 1] *= q_inv * g.y;
                v[k + 2] *= q_inv * g.z;
                v[k + 3] *= q_inv * g.w;
            }
            Vec<T>::store(cq + n * Rq + e, v);
        }
        return;
    }
    if (blockIdx.y == 0) {             // the query latent; the other block of the token stores
        for (int e = threadIdx.x; e < Rq; e += blockDim.x) {
            const float v = to_float(row[e]);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float q_inv = 1.0f / sqrtf(ss / (float)Rq + eps);
        for (int e = threadIdx.x; e < Rq; e += blockDim.x)
            cq[n * Rq + e] = from_float<T>(to_float(row[e]) * q_inv * q_gain[e]);
        return;
    }
    const int tr = token_row[n];
    if (!write || tr < 0) return;      // (uniform over the block)
    const int pos = positions[n];
    const int page = block_table[(int64_t)tr * table_stride + pos / page_size];
    if (page < 0) return;
    T* dst = pages + ((int64_t)page * page_size + pos % page_size) * Dp;
    const T* kv = row + kv_col;
    ss = 0.f;
    for (int e = threadIdx.x; e < R; e += blockDim.x) {
        const float v = to_float(kv[e]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float kv_inv = 1.0f / sqrtf(ss / (float)R + eps);
    for (int e = threadIdx.x; e < R; e += blockDim.x)
        dst[e] = from_float<T>(to_float(kv[e]) * kv_inv * kv_gain[e]);
    const int half = rot_dims / 2;
    const T* kr = kv + R;
    for (int e = threadIdx.x; e < Dp - R; e += blockDim.x) {
        float v = 0.f;
        if (e < rot_dims) {
            const int i = e < half ? e : e - half;
            const float c = cos_t[(int64_t)pos * half + i], s = sin_t[(int64_t)pos * half + i];
            const float u = to_float(kr[i]), w = to_float(kr[i + half]);
            v = e < half ? u * c - w * s : w * c + u * s;
        } else if (e < r) {
            v = to_float(kr[e]);
        }
        dst[R + e] = from_float<T>(v);
    }
}

// q: [N, H * (d + r)], head h's rotated part at column h * (d + r) + d; out: [N, H * Dp], the part
// lands at column h * Dp + R, zeros behind it up to Dp.  grid (N, ceil(H / heads per block)).
template <typename T>
__global__ void latent_q_rot_kernel(const T* __restrict__ q, int64_t ldq, int H, int d, int r,
                                    const int* __restrict__ positions,
                                    const float* __restrict__ cos_t,
                                    const float* __restrict__ sin_t, int rot_dims,
                                    T* __restrict__ out, int64_t ldo, int R, int Dp) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    const int pos = positions[n];
    const int half = rot_dims / 2, tail = Dp - R;
    for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < H * tail;
         idx += gridDim.y * blockDim.x) {
        const int h = idx / tail, e = idx - h * tail;
        const T* qr = q + n * ldq + (int64_t)h * (d + r) + d;
        float v = 0.f;
        if (e < rot_dims) {
            const int i = e < half ? e : e - half;
            const float c = cos_t[(int64_t)pos * half + i], s = sin_t[(int64_t)pos * half + i];
            const float u = to_float(qr[i]), w = to_float(qr[i + half]);
            v = e < half ? u * c - w * s : w * c + u * s;
        } else if (e < r) {
            v = to_float(qr[e]);
        }
        out[n * ldo + (int64_t)h * Dp + R + e] = from_float<T>(v);
    }
}

// out[n, h, j] = sum_k x[n, h, k] * w[h, j, k]: x rows at n * ldx + h * hsx, w [H, J, K]
// contiguous, out at n * ldo + h * hso + j.  Tiles of 32 tokens x 32 outputs of one head, k in
// steps of 16; every output is one chain of fused multiply-adds over k in ascending order, so
// a token's result depends on nothing else in the batch.  grid (ceil(J / 32), ceil(N / 32), H).
constexpr int HP_T = 32, HP_K = 16;
template <typename T>
__global__ void __launch_bounds__(256)
head_product_kernel(const T* __restrict__ x, int64_t ldx, int64_t hsx, const T* __restrict__ w,
                    T* __restrict__ out, int64_t ldo, int64_t hso, int N, int J, int K) {
    pdl_wait();
    pdl_trigger();
    __shared__ float xs[HP_K][HP_T + 1];
    __shared__ float ws[HP_K][HP_T + 1];
    const int h = blockIdx.z, n0 = blockIdx.y * HP_T, j0 = blockIdx.x * HP_T;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;   // 2 tokens x 2 outputs a thread
    const T* wh = w + (int64_t)h * J * K;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < K; k0 += HP_K) {
        for (int i = tid; i < HP_T * HP_K; i += 256) {
            const int t = i / HP_K, k = i - t * HP_K;
            xs[k][t] = (n0 + t < N && k0 + k < K)
                ? to_float(x[(int64_t)(n0 + t) * ldx + h * hsx + k0 + k]) : 0.f;
            ws[k][t] = (j0 + t < J && k0 + k < K)
                ? to_float(wh[(int64_t)(j0 + t) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HP_K; ++k) {
            const float a0 = xs[k][ty * 2], a1 = xs[k][ty * 2 + 1];
            const float b0 = ws[k][tx * 2], b1 = ws[k][tx * 2 + 1];
            acc[0][0] = fmaf(a0, b0, acc[0][0]);
            acc[0][1] = fmaf(a0, b1, acc[0][1]);
            acc[1][0] = fmaf(a1, b0, acc[1][0]);
            acc[1][1] = fmaf(a1, b1, acc[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int n = n0 + ty * 2 + i, c = j0 + tx * 2 + j;
            if (n < N && c < J)
                out[(int64_t)n * ldo + h * hso + c] = from_float<T>(acc[i][j]);
        }
}

// x[n, h * V + j] *= sigmoid(gate[n * ldg + h]).  One block per token.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, int64_t ldx, const T* __restrict__ gate,
                                 int64_t ldg, int H, int V) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    for (int idx = threadIdx.x; idx < H * V; idx += blockDim.x) {
        const float g = to_float(gate[n * ldg + idx / V]);
        T* p = x + n * ldx + idx;
        *p = from_float<T>(to_float(*p) / (1.0f + expf(-g)));
    }
}

// head_gate_kernel with 16-byte accesses (V a multiple of Vec<T>::N, rows 16-byte aligned):
// a thread's vector lies within one head.  grid (N, ceil(H * V / (N * 256))).
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_vec_kernel(T* __restrict__ x, int64_t ldx, const T* __restrict__ gate, int64_t ldg,
                     int H, int V) {
    pdl_wait();
    pdl_trigger();
    constexpr int VN = Vec<T>::N;
    const int64_t n = blockIdx.x;
    const int idx = (blockIdx.y * 256 + threadIdx.x) * VN;
    if (idx >= H * V) return;
    const float g = to_float(gate[n * ldg + idx / V]);
    const float f = 1.0f / (1.0f + expf(-g));
    float v[VN];
    Vec<T>::load(x + n * ldx + idx, v);
#pragma unroll
    for (int i = 0; i < VN; ++i) v[i] *= f;
    Vec<T>::store(x + n * ldx + idx, v);
}

// latent_q_rot_kernel with 16-byte accesses: d, r, R, the tail Dp - R and rot_dims / 2 are
// multiples of Vec<T>::N and rows are 16-byte aligned, so a thread's vector of the tail is
// wholly in the rotation's first half, its second half, the unrotated rest or the zeros.
// grid (N, ceil(H * tail / (N * 256))).
template <typename T>
__global__ void __launch_bounds__(256)
latent_q_rot_vec_kernel(const T* __restrict__ q, int64_t ldq, int H, int d, int r,
                        const int* __restrict__ positions, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, int rot_dims, T* __restrict__ out,
                        int64_t ldo, int R, int Dp) {
    pdl_wait();
    pdl_trigger();
    constexpr int VN = Vec<T>::N;
    const int64_t n = blockIdx.x;
    const int tail = Dp - R, half = rot_dims / 2;
    const int idx = (blockIdx.y * 256 + threadIdx.x) * VN;
    if (idx >= H * tail) return;
    const int h = idx / tail, e = idx - h * tail;
    const T* qr = q + n * ldq + (int64_t)h * (d + r) + d;
    float v[VN];
    if (e < rot_dims) {
        const int i = e < half ? e : e - half;
        const int64_t at = (int64_t)positions[n] * half + i;
        float u[VN], w[VN];
        Vec<T>::load(qr + i, u);
        Vec<T>::load(qr + i + half, w);
#pragma unroll
        for (int k = 0; k < VN; k += 4) {
            const float4 c = *reinterpret_cast<const float4*>(cos_t + at + k);
            const float4 sn = *reinterpret_cast<const float4*>(sin_t + at + k);
            const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
            for (int m = 0; m < 4; ++m)
                v[k + m] = e < half ? u[k + m] * cc[m] - w[k + m] * ss[m]
                                    : w[k + m] * cc[m] + u[k + m] * ss[m];
        }
    } else if (e < r) {
        Vec<T>::load(qr + e, v);
    } else {
#pragma unroll
        for (int k = 0; k < VN; ++k) v[k] = 0.f;
    }
    Vec<T>::store(out + n * ldo + (int64_t)h * Dp + R + e, v);
}

// Steps of few tokens: out[n, h, j] = f(n, h) * sum_k x[n, h, k] * w[h, k, j], with w [H, K, J]
// (the output index last, so that a warp reads a row of w at a time).  A CTA has LS_T tokens of
// one head and LS_J neighbouring outputs: grid (H, ceil(N / LS_T), ceil(J / LS_J)), 256 threads,
// the tile's x rows in shared memory as 32-bit.  Warp g takes the reduction indices g, g + 8, ...
// (a lane is an output) and requests eight rows of w at a time; the eight partial sums of an
// output meet in shared memory and are added in the order of the warps, so a token's result
// depends on nothing else in the batch.  The matrices of a step are small (H K J entries), so
// what counts is that enough CTAs have enough loads in flight.  Options: `gate` (f = sigmoid of
// gate[n * ldg + h], else 1), and a rotated tail as latent_q_rot_kernel writes it (the head's
// entries K .. K + r of x, rotated, at out columns J .. J + tail, zeros behind the r), which the
// CTAs of the first outputs write.
constexpr int LS_T = 8;
constexpr int LS_J = 32;
constexpr int LS_G = 8;
static_assert(LS_G == LS_T && LS_G * 32 == 256 && LS_J == 32, "a warp per reduction group and per token");
template <typename T>
__global__ void __launch_bounds__(256)
latent_small_kernel(const T* __restrict__ x, int64_t ldx, int64_t hsx, const T* __restrict__ w,
                    T* __restrict__ out, int64_t ldo, int64_t hso, int N, int K, int J,
                    const T* __restrict__ gate, int64_t ldg, int r, int tail,
                    const int* __restrict__ positions, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, int rot_dims) {
    extern __shared__ float ls_smem[];
    const int h = blockIdx.x, n0 = blockIdx.y * LS_T, tid = threadIdx.x;
    const int g = tid >> 5, lane = tid & 31;
    const int j = blockIdx.z * LS_J + lane;
    const int nt = min(LS_T, N - n0);
    float* xs = ls_smem;                       // [LS_T][K]
    float* red = ls_smem + LS_T * K;           // [LS_G][LS_T][LS_J]
    // the matrix does not depend on the kernel before: its first rows are requested ahead of it
    const T* wj = w + (int64_t)h * K * J + (j < J ? j : 0);
    T wv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int k = g + u * LS_G;
        wv[u] = k < K ? wj[(int64_t)k * J] : from_float<T>(0.f);
    }
    pdl_wait();
    pdl_trigger();
    for (int i = tid; i < LS_T * K; i += 256) {
        const int t = i / K, k = i - t * K;
        xs[i] = t < nt ? to_float(x[(int64_t)(n0 + t) * ldx + h * hsx + k]) : 0.f;
    }
    __syncthreads();
    float acc[LS_T];
#pragma unroll
    for (int t = 0; t < LS_T; ++t) acc[t] = 0.f;
    for (int k0 = g; k0 < K; k0 += 8 * LS_G) {
        T nx[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {           // the next eight rows, before these are used
            const int k = k0 + (8 + u) * LS_G;
            nx[u] = k < K ? wj[(int64_t)k * J] : from_float<T>(0.f);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int k = k0 + u * LS_G;
            if (k < K) {
                const float wf = to_float(wv[u]);
#pragma unroll
                for (int t = 0; t < LS_T; ++t) acc[t] = fmaf(xs[t * K + k], wf, acc[t]);
            }
            wv[u] = nx[u];
        }
    }
#pragma unroll
    for (int t = 0; t < LS_T; ++t) red[(g * LS_T + t) * LS_J + lane] = acc[t];
    __syncthreads();
    {   // thread (token g, output lane): the partial sums in the order of the warps
        const int t = g;
        float sum = red[t * LS_J + lane];
#pragma unroll
        for (int gg = 1; gg < LS_G; ++gg) sum += red[(gg * LS_T + t) * LS_J + lane];
        if (t < nt && j < J) {
            float f = 1.f;
            if (gate) f = 1.0f / (1.0f + expf(-to_float(gate[(int64_t)(n0 + t) * ldg + h])));
            out[(int64_t)(n0 + t) * ldo + h * hso + j] = from_float<T>(sum * f);
        }
    }
    if (tail <= 0 || blockIdx.z != 0) return;
    const int half = rot_dims / 2;
    for (int idx = tid; idx < nt * tail; idx += 256) {
        const int t = idx / tail, e = idx - t * tail;
        const int pos = positions[n0 + t];
        const T* qr = x + (int64_t)(n0 + t) * ldx + h * hsx + K;
        float v = 0.f;
        if (e < rot_dims) {
            const int i = e < half ? e : e - half;
            const float c = cos_t[(int64_t)pos * half + i], sn = sin_t[(int64_t)pos * half + i];
            const float u = to_float(qr[i]), ww = to_float(qr[i + half]);
            v = e < half ? u * c - ww * sn : ww * c + u * sn;
        } else if (e < r) {
            v = to_float(qr[e]);
        }
        out[(int64_t)(n0 + t) * ldo + h * hso + J + e] = from_float<T>(v);
    }
}

}  // namespace sllm

using namespace sllm;

// pages: [n_pages, 1, 1, page_size, Dp].  cos_t / sin_t: float [positions, rot_dims / 2].
SLLM_EXPORT int sllm_latent_prep(const void* a, int64_t lda, int Rq, int kv_col, int R, int r,
                                 const float* q_gain, const float* kv_gain, float eps,
                                 const int* positions, const int* token_row, const float* cos_t,
                                 const float* sin_t, int rot_dims, void* cq, void* pages,
                                 const int* block_table, int table_stride, int page_size, int Dp,
                                 int write, int n_tokens, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (Rq < 1 || R < 1 || r < 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > r ||
        Dp < R + r || page_size < 1 || kv_col < 0)
        return (int)cudaErrorInvalidValue;
    typedef __nv_bfloat16 bf16;
    // the query latent moves 16 bytes at a time where its rows allow it
    const int vn = dtype == 0 ? 4 : 8;
    const int vec = Rq % vn == 0 && lda % vn == 0 &&
                    !(((uintptr_t)a | (uintptr_t)cq | (uintptr_t)q_gain) & 15);
    if (dtype == 0)
        return (int)sllm_launch_pdl(latent_prep_kernel<float>, dim3(n_tokens, 2), dim3(256), 0, stream,
                                    (const float*)a, lda, Rq, kv_col, R, r, q_gain, kv_gain, eps,
                                    positions, token_row, cos_t, sin_t, rot_dims, (float*)cq,
                                    (float*)pages, block_table, table_stride, page_size, Dp, write, vec);
    if (dtype == 1)
        return (int)sllm_launch_pdl(latent_prep_kernel<bf16>, dim3(n_tokens, 2), dim3(256), 0, stream,
                                    (const bf16*)a, lda, Rq, kv_col, R, r, q_gain, kv_gain, eps,
                                    positions, token_row, cos_t, sin_t, rot_dims, (bf16*)cq,
                                    (bf16*)pages, block_table, table_stride, page_size, Dp, write, vec);
    return (int)cudaErrorInvalidValue;
}

SLLM_EXPORT int sllm_latent_q_rot(const void* q, int64_t ldq, int H, int d, int r,
                                  const int* positions, const float* cos_t, const float* sin_t,
                                  int rot_dims, void* out, int64_t ldo, int R, int Dp,
                                  int n_tokens, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || Dp == R) return 0;
    if (H < 1 || d < 0 || r < 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > r || Dp < R + r)
        return (int)cudaErrorInvalidValue;
    const int work = H * (Dp - R);
    typedef __nv_bfloat16 bf16;
    const int vn = dtype == 0 ? 4 : 8;
    if ((d | r | R | Dp | (rot_dims / 2)) % vn == 0 && ldq % vn == 0 && ldo % vn == 0 &&
        !(((uintptr_t)q | (uintptr_t)out | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) &&
        (work / vn + 255) / 256 <= 65535 && dtype >= 0 && dtype <= 1) {
        dim3 vgrid(n_tokens, (work / vn + 255) / 256);
        if (dtype == 0)
            return (int)sllm_launch_pdl(latent_q_rot_vec_kernel<float>, vgrid, dim3(256), 0, stream,
                                        (const float*)q, ldq, H, d, r, positions, cos_t, sin_t,
                                        rot_dims, (float*)out, ldo, R, Dp);
        return (int)sllm_launch_pdl(latent_q_rot_vec_kernel<bf16>, vgrid, dim3(256), 0, stream,
                                    (const bf16*)q, ldq, H, d, r, positions, cos_t, sin_t,
                                    rot_dims, (bf16*)out, ldo, R, Dp);
    }
    dim3 grid(n_tokens, (work + 255) / 256 > 8 ? 8 : (work + 255) / 256);
    if (dtype == 0)
        return (int)sllm_launch_pdl(latent_q_rot_kernel<float>, grid, dim3(256), 0, stream,
                                    (const float*)q, ldq, H, d, r, positions, cos_t, sin_t,
                                    rot_dims, (float*)out, ldo, R, Dp);
    if (dtype == 1)
        return (int)sllm_launch_pdl(latent_q_rot_kernel<bf16>, grid, dim3(256), 0, stream,
                                    (const bf16*)q, ldq, H, d, r, positions, cos_t, sin_t,
                                    rot_dims, (bf16*)out, ldo, R, Dp);
    return (int)cudaErrorInvalidValue;
}

SLLM_EXPORT int sllm_head_product(const void* x, int64_t ldx, int64_t hsx, const void* w, void* out,
                                  int64_t ldo, int64_t hso, int n_tokens, int H, int J, int K,
                                  int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H < 1 || H > 65535 || J < 1 || K < 1 || (n_tokens + HP_T - 1) / HP_T > 65535)
        return (int)cudaErrorInvalidValue;
    dim3 grid((J + HP_T - 1) / HP_T, (n_tokens + HP_T - 1) / HP_T, H);
    typedef __nv_bfloat16 bf16;
    if (dtype == 0)
        return (int)sllm_launch_pdl(head_product_kernel<float>, grid, dim3(256), 0, stream,
                                    (const float*)x, ldx, hsx, (const float*)w, (float*)out, ldo,
                                    hso, n_tokens, J, K);
    if (dtype == 1)
        return (int)sllm_launch_pdl(head_product_kernel<bf16>, grid, dim3(256), 0, stream,
                                    (const bf16*)x, ldx, hsx, (const bf16*)w, (bf16*)out, ldo, hso,
                                    n_tokens, J, K);
    return (int)cudaErrorInvalidValue;
}

SLLM_EXPORT int sllm_head_gate(void* x, int64_t ldx, const void* gate, int64_t ldg, int H, int V,
                               int n_tokens, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H < 1 || V < 1) return (int)cudaErrorInvalidValue;
    typedef __nv_bfloat16 bf16;
    const int vn = dtype == 0 ? 4 : 8;
    if (V % vn == 0 && ldx % vn == 0 && !((uintptr_t)x & 15) && dtype >= 0 && dtype <= 1 &&
        (H * V / vn + 255) / 256 <= 65535) {
        dim3 vgrid(n_tokens, (H * V / vn + 255) / 256);
        if (dtype == 0)
            return (int)sllm_launch_pdl(head_gate_vec_kernel<float>, vgrid, dim3(256), 0, stream,
                                        (float*)x, ldx, (const float*)gate, ldg, H, V);
        return (int)sllm_launch_pdl(head_gate_vec_kernel<bf16>, vgrid, dim3(256), 0, stream,
                                    (bf16*)x, ldx, (const bf16*)gate, ldg, H, V);
    }
    if (dtype == 0)
        return (int)sllm_launch_pdl(head_gate_kernel<float>, dim3(n_tokens), dim3(256), 0, stream,
                                    (float*)x, ldx, (const float*)gate, ldg, H, V);
    if (dtype == 1)
        return (int)sllm_launch_pdl(head_gate_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream,
                                    (bf16*)x, ldx, (const bf16*)gate, ldg, H, V);
    return (int)cudaErrorInvalidValue;
}

// Steps of few tokens (see latent_small_kernel).  gate may be null; tail 0 leaves the rotated
// part out (then r, positions and the tables are unused).
SLLM_EXPORT int sllm_latent_small(const void* x, int64_t ldx, int64_t hsx, const void* w, void* out,
                                  int64_t ldo, int64_t hso, int n_tokens, int H, int K, int J,
                                  const void* gate, int64_t ldg, int r, int tail,
                                  const int* positions, const float* cos_t, const float* sin_t,
                                  int rot_dims, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H < 1 || H > 65535 || K < 1 || J < 1 || r < 0 || tail < 0 || (tail && tail < r) ||
        rot_dims < 0 || (rot_dims & 1) || rot_dims > r || (n_tokens + LS_T - 1) / LS_T > 65535)
        return (int)cudaErrorInvalidValue;
    const size_t smem = sizeof(float) * ((size_t)LS_T * K + (size_t)LS_G * LS_T * LS_J);
    if (smem > 48 * 1024 || (J + LS_J - 1) / LS_J > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid(H, (n_tokens + LS_T - 1) / LS_T, (J + LS_J - 1) / LS_J);
    typedef __nv_bfloat16 bf16;
    if (dtype == 0)
        return (int)sllm_launch_pdl(latent_small_kernel<float>, grid, dim3(256), smem, stream,
                                    (const float*)x, ldx, hsx, (const float*)w, (float*)out, ldo,
                                    hso, n_tokens, K, J, (const float*)gate, ldg, r, tail,
                                    positions, cos_t, sin_t, rot_dims);
    if (dtype == 1)
        return (int)sllm_launch_pdl(latent_small_kernel<bf16>, grid, dim3(256), smem, stream,
                                    (const bf16*)x, ldx, hsx, (const bf16*)w, (bf16*)out, ldo, hso,
                                    n_tokens, K, J, (const bf16*)gate, ldg, r, tail, positions,
                                    cos_t, sin_t, rot_dims);
    return (int)cudaErrorInvalidValue;
}
