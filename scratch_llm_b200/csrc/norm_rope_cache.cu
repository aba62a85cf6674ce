// What stands between an attention mixer's fused projection and its attention kernel, for
// designs that norm their queries and keys: biases, an RMS norm over the whole projection
// before the rotation, the rotation, an RMS norm per head after it, and the write of the new
// keys and values into the paged cache.  Every step is optional.
//
// x is [n_tokens, ld]: H query heads, then (if the projection has them) G key heads and G value
// heads, each `hd` wide, then whatever else the fused projection holds (not touched).  Heads
// may be padded with zero columns beyond their true size `qk_dim` (the kernels and the cache
// have one head size); the norms divide by the true sizes.
//
//   q, k, v  +=  bias                                             (bias != null)
//   q  <-  q / sqrt(sum(q^2) / (H qk_dim) + eps) * q_gain         (q_gain != null: over ALL heads
//   k  <-  k / sqrt(sum(k^2) / (G qk_dim) + eps) * k_gain          at once, gains per column)
//   q, k  <-  rotated by the position's angles                    (cos_t != null; tables of
//                                                                  rot / 2 columns, pairs (2i,
//                                                                  2i+1) or (i, i + rot/2))
//   q[h], k[g]  <-  / sqrt(mean over qk_dim of the head's squares + eps)     (unit_after)
//   q back in place; K page <- k, V page <- v                     (has_kv and write)
//
// pages: [n_pages, 2 (K, V), G, page_size, hd]; page = block_table[row, p / page_size].
// A token whose row is -1 is padding: nothing of it is touched.  All arithmetic is 32-bit on a
// copy of the token's row in shared memory, with one rounding at the end.
#include "common.cuh"

namespace sllm {

constexpr int NR_THREADS = 256;

struct NormRopeArgs {
    void* x; int64_t ld;
    const int* positions; const int* token_row;
    const float* bias; const float* q_gain; const float* k_gain;
    int unit_after; float eps; int qk_dim;
    const float* cos_t; const float* sin_t; int rot; int interleaved;
    void* pages; const int* block_table; int table_stride; int page_size;
    int H; int G; int hd; int has_kv; int write;
};

// VECTOR: the token's columns come and go 16 bytes at a time (hd a multiple of 16 / sizeof(T),
// rows and bases 16-byte aligned); the arithmetic in between is the same.
template <typename T, bool VECTOR>
__global__ void __launch_bounds__(NR_THREADS) norm_rope_kv_write_kernel(const NormRopeArgs a) {
    extern __shared__ __align__(16) float s[];        // the token's q (and k, v) columns
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    const int row = a.token_row[n];
    if (row < 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = a.hd;
    const bool kv = a.has_kv && a.write;
    const int q_cols = a.H * hd, k_cols = kv ? a.G * hd : 0;
    const int cols = q_cols + 2 * k_cols;
    T* x = reinterpret_cast<T*>(a.x) + n * a.ld;
    constexpr int VN = Vec<T>::N;
    if (VECTOR) {
        for (int c = tid * VN; c < cols; c += NR_THREADS * VN) {
            float v[VN];
            Vec<T>::load(x + c, v);
#pragma unroll
            for (int i = 0; i < VN; ++i) s[c + i] = v[i] + (a.bias ? a.bias[c + i] : 0.f);
        }
    } else {
        for (int c = tid; c < cols; c += NR_THREADS)
            s[c] = to_float(x[c]) + (a.bias ? a.bias[c] : 0.f);
    }
    __syncthreads();
    if (a.q_gain) {     // one factor for all of q, one for all of k
        float sq = 0.f, sk = 0.f;
        for (int c = tid; c < q_cols; c += NR_THREADS) sq = fmaf(s[c], s[c], sq);
        for (int c = tid; c < k_cols; c += NR_THREADS) sk = fmaf(s[q_cols + c], s[q_cols + c], sk);
        sq = block_sum(sq, scratch);
        sk = block_sum(sk, scratch);
        const float iq = 1.0f / sqrtf(sq / (float)(a.H * a.qk_dim) + a.eps);
        const float ik = 1.0f / sqrtf(sk / (float)(a.G * a.qk_dim) + a.eps);
        for (int c = tid; c < q_cols; c += NR_THREADS) s[c] *= iq * a.q_gain[c];
        for (int c = tid; c < k_cols; c += NR_THREADS) s[q_cols + c] *= ik * a.k_gain[c];
        __syncthreads();
    }
    const int heads = a.H + (kv ? a.G : 0);     // q heads, then k heads: contiguous in s
    if (a.cos_t) {
        const int half = a.rot >> 1;
        const int pos = a.positions[n];
        const float* ct = a.cos_t + (int64_t)pos * half;
        const float* st = a.sin_t + (int64_t)pos * half;
        for (int idx = tid; idx < heads * half; idx += NR_THREADS) {
            const int head = idx / half, i = idx - head * half;
            float* h = s + head * hd;
            const int ia = a.interleaved ? 2 * i : i, ib = a.interleaved ? 2 * i + 1 : i + half;
            const float u = h[ia], v = h[ib], c = ct[i], sn = st[i];
            h[ia] = u * c - v * sn;
            h[ib] = v * c + u * sn;
        }
        __syncthreads();
    }
    if (a.unit_after) {
        for (int head = warp; head < heads; head += NR_THREADS / 32) {
            float* h = s + head * hd;
            float ss = 0.f;
            for (int d = lane; d < hd; d += 32) ss = fmaf(h[d], h[d], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)a.qk_dim + a.eps);
            for (int d = lane; d < hd; d += 32) h[d] *= inv;
        }
        __syncthreads();
    }
    if (VECTOR) {
        for (int c = tid * VN; c < q_cols; c += NR_THREADS * VN) Vec<T>::store(x + c, s + c);
    } else {
        for (int c = tid; c < q_cols; c += NR_THREADS) x[c] = from_float<T>(s[c]);
    }
    if (!kv) return;
    const int pos = a.positions[n];
    const int page = a.block_table[(int64_t)row * a.table_stride + pos / a.page_size];
    if (page < 0) return;
    T* pages = reinterpret_cast<T*>(a.pages);
    const int64_t plane = (int64_t)a.G * a.page_size * hd;
    T* k_dst = pages + (int64_t)page * 2 * plane + (int64_t)(pos % a.page_size) * hd;
    if (VECTOR) {
        for (int c = tid * VN; c < k_cols; c += NR_THREADS * VN) {
            const int g = c / hd, d = c - g * hd;
            const int64_t off = (int64_t)g * a.page_size * hd + d;
            Vec<T>::store(k_dst + off, s + q_cols + c);
            Vec<T>::store(k_dst + plane + off, s + q_cols + k_cols + c);
        }
    } else {
        for (int c = tid; c < k_cols; c += NR_THREADS) {
            const int g = c / hd, d = c - g * hd;
            const int64_t off = (int64_t)g * a.page_size * hd + d;
            k_dst[off] = from_float<T>(s[q_cols + c]);
            k_dst[plane + off] = from_float<T>(s[q_cols + k_cols + c]);
        }
    }
}

}  // namespace sllm

using namespace sllm;

// dtype: 0 = float32, 1 = bfloat16 (of x and pages).  bias (may be null): float
// [(H + 2 G) * hd], or [H * hd] without has_kv.  q_gain / k_gain (both or neither; k_gain may be
// null without has_kv): float [H * hd] / [G * hd].  cos_t / sin_t (may be null): float
// [positions, rot / 2].
SLLM_EXPORT int sllm_norm_rope_kv_write(void* x, int64_t ld, const int* positions,
                                        const int* token_row, const float* bias,
                                        const float* q_gain, const float* k_gain, int unit_after,
                                        float eps, int qk_dim, const float* cos_t,
                                        const float* sin_t, int rot, int interleaved, void* pages,
                                        const int* block_table, int table_stride, int page_size,
                                        int n_tokens, int H, int G, int hd, int has_kv, int write,
                                        int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || hd <= 0 || qk_dim <= 0 || qk_dim > hd || page_size <= 0 ||
        ld < (int64_t)(H + (has_kv ? 2 * G : 0)) * hd || (cos_t && (rot < 2 || rot % 2 || rot > qk_dim)) ||
        (cos_t != nullptr) != (sin_t != nullptr) || (has_kv && q_gain && !k_gain))
        return (int)cudaErrorInvalidValue;
    NormRopeArgs a;
    a.x = x; a.ld = ld; a.positions = positions; a.token_row = token_row; a.bias = bias;
    a.q_gain = q_gain; a.k_gain = k_gain; a.unit_after = unit_after; a.eps = eps;
    a.qk_dim = qk_dim; a.cos_t = cos_t; a.sin_t = sin_t; a.rot = rot; a.interleaved = interleaved;
    a.pages = pages; a.block_table = block_table; a.table_stride = table_stride;
    a.page_size = page_size; a.H = H; a.G = G; a.hd = hd; a.has_kv = has_kv; a.write = write;
    const size_t smem = (size_t)(H + (has_kv ? 2 * G : 0)) * hd * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (dtype != 0 && dtype != 1) return (int)cudaErrorInvalidValue;
    const int vn = dtype == 0 ? 4 : 8;
    const bool vector = hd % vn == 0 && ld % vn == 0 && !(((uintptr_t)x | (uintptr_t)pages) & 15);
    cudaError_t e = cudaSuccess;
#define SLLM_NR_LAUNCH(T, V)                                                                   \
    do {                                                                                       \
        if (smem > 48 * 1024) {                                                                \
            e = cudaFuncSetAttribute(norm_rope_kv_write_kernel<T, V>,                          \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
            if (e != cudaSuccess) return (int)e;                                               \
        }                                                                                      \
        e = sllm_launch_pdl(norm_rope_kv_write_kernel<T, V>, dim3(n_tokens), dim3(NR_THREADS), \
                            smem, stream, a);                                                  \
    } while (0)
    if (dtype == 0) {
        if (vector) SLLM_NR_LAUNCH(float, true); else SLLM_NR_LAUNCH(float, false);
    } else {
        if (vector) SLLM_NR_LAUNCH(__nv_bfloat16, true); else SLLM_NR_LAUNCH(__nv_bfloat16, false);
    }
#undef SLLM_NR_LAUNCH
    return (int)e;
}
