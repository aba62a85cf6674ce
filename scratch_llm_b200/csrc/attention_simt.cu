// Causal attention of a packed batch over the paged cache, on the CUDA cores in 32-bit
// arithmetic.  One kernel serves portions of prompts and single decoded tokens: the token at
// absolute position p of row r attends to keys 0..p of row r (or to the last `window` of
// them) through r's block table.  This is the attention of the 32-bit path for every head
// size, and of the bfloat16 path where no tensor-core kernel takes the shape.
//
// Restates src/scratch_llm/model.py:172-182 (scores = q k^T scaled, disallowed keys -inf,
// max-subtracted softmax in 32-bit, times v) and :330-345 (query head h reads kv head
// h / (H/G); key j is visible to the query at position p iff j <= p) of the reference, with
// the online softmax of its paged kernel (src/scratch_llm/kernels/attention/decode/paged.py:49-83).
//
// Keys are consumed in tiles of 32 that are aligned to absolute positions, in ascending
// order, so a query's result does not depend on how its prompt was cut or on its neighbours.
// Compiled once per head size: -DSLLM_HEAD_DIM=<1 to 640>.
#include "common.cuh"

#ifndef SLLM_HEAD_DIM
#error "compile with -DSLLM_HEAD_DIM=<head size>"
#endif

namespace sllm {

constexpr int HD = SLLM_HEAD_DIM;
static_assert(HD >= 1 && HD <= 640, "head size: 1 to 640");
constexpr int BQ = 16, BKV = 32, THREADS = 128, ROWS_PER_WARP = 4;
constexpr int DPL = (HD + 31) / 32;  // head dims per lane
constexpr int KS_LD = HD + 1;

constexpr size_t smem_floats() {
    return (size_t)BQ * HD + (size_t)BKV * KS_LD + (size_t)BKV * HD + (size_t)BQ * BKV;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_simt_kernel(const T* __restrict__ q, int64_t q_stride, const T* __restrict__ pages,
                 const int* __restrict__ block_table, int table_stride, int page_size,
                 const int* __restrict__ row_start, const int* __restrict__ row_pos0,
                 T* __restrict__ out, int64_t out_stride, int H, int G, float scale, int window,
                 const float* __restrict__ slopes, const float* __restrict__ sinks, int planes,
                 float softcap, int chunk) {
    extern __shared__ float smem[];
    __shared__ long long key_base[BKV];  // element offset of each key's K row, -1 if absent
    float* Qs = smem;
    float* Ks = Qs + BQ * HD;
    float* Vs = Ks + BKV * KS_LD;
    float* Ss = Vs + BKV * HD;

    const int r = blockIdx.y, h = blockIdx.z;
    const int g = h / (H / G);
    const int t0 = row_start[r];
    const int n_new = row_start[r + 1] - t0;
    const int q0 = blockIdx.x * BQ;
    if (q0 >= n_new) return;
    const int nq = min(BQ, n_new - q0);
    const int first_pos = row_pos0[r] + q0;
    const int last_pos = first_pos + nq - 1;
    int k_lo = 0;
    if (window > 0) k_lo = max(0, first_pos - window + 1) / BKV * BKV;
    if (chunk > 0) k_lo = max(k_lo, first_pos / chunk * chunk / BKV * BKV);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float slope = slopes ? slopes[h] : 0.f;

    for (int idx = tid; idx < BQ * HD; idx += THREADS) {
        const int i = idx / HD, d = idx - i * HD;
        Qs[idx] = i < nq ? to_float(q[(int64_t)(t0 + q0 + i) * q_stride + (int64_t)h * HD + d])
                         : 0.f;
    }

    float m[ROWS_PER_WARP], l[ROWS_PER_WARP], acc[ROWS_PER_WARP][DPL];
#pragma unroll
    for (int a = 0; a < ROWS_PER_WARP; ++a) {
        m[a] = -INFINITY;
        l[a] = 0.f;
#pragma unroll
        for (int c = 0; c < DPL; ++c) acc[a][c] = 0.f;
    }
    // (one plane: the values are the leading entries of the keys themselves)
    const int64_t v_offset = (int64_t)(planes - 1) * G * page_size * HD;

    for (int kt = k_lo; kt <= last_pos; kt += BKV) {
        __syncthreads();  // the previous tile's Ks / Vs / key_base are no longer read
        if (tid < BKV) {
            const int kpos = kt + tid;
            long long base = -1;
            if (kpos <= last_pos) {
                const int page = block_table[(int64_t)r * table_stride + kpos / page_size];
                if (page >= 0)
                    base = (((long long)page * planes * G + g) * page_size + kpos % page_size) * HD;
            }
            key_base[tid] = base;
        }
        __syncthreads();
        for (int idx = tid; idx < BKV * HD; idx += THREADS) {
            const int j = idx / HD, d = idx - j * HD;
            const long long base = key_base[j];
            float kv = 0.f, vv = 0.f;
            if (base >= 0) {
                kv = to_float(pages[base + d]);
                vv = to_float(pages[base + v_offset + d]);
            }
            Ks[j * KS_LD + d] = kv;
            Vs[j * HD + d] = vv;
        }
        __syncthreads();

        const int kpos = kt + lane;
#pragma unroll
        for (int a = 0; a < ROWS_PER_WARP; ++a) {
            const int i = warp + 4 * a;
            const float* qi = Qs + i * HD;
            const float* kj = Ks + lane * KS_LD;
            float dot = 0.f;
#pragma unroll 8
            for (int d = 0; d < HD; ++d) dot = fmaf(qi[d], kj[d], dot);
            const int qpos = first_pos + i;
            const bool valid = i < nq && kpos <= qpos && (window <= 0 || kpos > qpos - window) &&
                               (chunk <= 0 || kpos >= qpos / chunk * chunk) && key_base[lane] >= 0;
            float sc = dot * scale;
            if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
            const float s = valid ? sc - slope * (float)(qpos - kpos) : -INFINITY;
            const float m_new = fmaxf(m[a], warp_max(s));
            float p = 0.f, corr = 1.f;
            if (m_new != -INFINITY) {
                p = expf(s - m_new);        // s = -inf gives 0
                corr = expf(m[a] - m_new);  // m = -inf gives 0
            }
            l[a] = l[a] * corr + warp_sum(p);
            m[a] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) acc[a][c] *= corr;
            Ss[i * BKV + lane] = p;
        }
        __syncwarp();  // each warp reads back only the rows of Ss it wrote
#pragma unroll
        for (int a = 0; a < ROWS_PER_WARP; ++a) {
            const float* pi = Ss + (warp + 4 * a) * BKV;
            for (int j = 0; j < BKV; ++j) {
                const float p = pi[j];
#pragma unroll
                for (int c = 0; c < DPL; ++c) {
                    const int d = lane + 32 * c;
                    if (d < HD) acc[a][c] = fmaf(p, Vs[j * HD + d], acc[a][c]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < ROWS_PER_WARP; ++a) {
        const int i = warp + 4 * a;
        if (i >= nq) continue;
        float total = l[a], keep = 1.f;
        if (sinks && m[a] != -INFINITY) {
            // the sink: one more term of the denominator, without a key or a value
            const float sink = sinks[h], top = fmaxf(m[a], sink);
            keep = expf(m[a] - top);
            total = total * keep + expf(sink - top);
        }
        const float inv = total > 0.f ? keep / total : 0.f;
        T* o = out + (int64_t)(t0 + q0 + i) * out_stride + (int64_t)h * HD;
#pragma unroll
        for (int c = 0; c < DPL; ++c) {
            const int d = lane + 32 * c;
            if (d < HD) o[d] = from_float<T>(acc[a][c] * inv);
        }
    }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_attn_simt_head_dim() { return HD; }

// q: [n_tokens, q_stride] with head h at columns [h*HD, (h+1)*HD); out likewise.
// pages: [n_pages, planes, G, page_size, HD]; planes = 2: keys, then values; planes = 1: one
// vector per token that is its key and, by its leading entries, its value.  block_table: [n_rows, table_stride], -1 = no page.
// row_start: [n_rows + 1] token offsets; row_pos0: [n_rows] position of each row's first token.
// max_new: the largest number of new tokens of any row.  window: 0 = all keys.
// slopes (may be null): float [H]; slopes[h] * (query position - key position) is taken off the
// scaled score of head h.  sinks (may be null): float [H]; exp(sinks[h]) is added to the softmax's
// denominator of head h, once, with no value behind it.  softcap > 0: the scaled score s becomes
// softcap * tanh(s / softcap) (before the slopes).  chunk > 0: the query at position p sees only
// keys from floor(p / chunk) * chunk on (positions count from the sequence's start).
SLLM_EXPORT int sllm_attn_simt(const void* q, int64_t q_stride, const void* pages,
                               const int* block_table, int table_stride, int page_size,
                               const int* row_start, const int* row_pos0, void* out,
                               int64_t out_stride, int n_rows, int max_new, int H, int G,
                               float scale, int window, const float* slopes, const float* sinks,
                               int planes, float softcap, int chunk, int dtype,
                               cudaStream_t stream) {
    if (n_rows <= 0 || max_new <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || page_size <= 0 || window < 0 || chunk < 0 || planes < 1 || planes > 2)
        return (int)cudaErrorInvalidValue;
    if (n_rows > 65535 || H > 65535) return (int)cudaErrorInvalidValue;
    const size_t smem = smem_floats() * sizeof(float);
    dim3 grid((max_new + BQ - 1) / BQ, n_rows, H);
    cudaError_t e;
    if (dtype == 0) {
        e = cudaFuncSetAttribute(attn_simt_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attn_simt_kernel<float><<<grid, THREADS, smem, stream>>>(
            (const float*)q, q_stride, (const float*)pages, block_table, table_stride, page_size,
            row_start, row_pos0, (float*)out, out_stride, H, G, scale, window, slopes, sinks,
            planes, softcap, chunk);
    } else if (dtype == 1) {
        e = cudaFuncSetAttribute(attn_simt_kernel<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attn_simt_kernel<__nv_bfloat16><<<grid, THREADS, smem, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)pages, block_table,
            table_stride, page_size, row_start, row_pos0, (__nv_bfloat16*)out, out_stride, H, G,
            scale, window, slopes, sinks, planes, softcap, chunk);
    } else {
        return (int)cudaErrorInvalidValue;
    }
    SLLM_LAUNCH_CHECK();
    return 0;
}
