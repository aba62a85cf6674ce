// A routed feed-forward (mixture of experts) without a host round trip, so that its steps can
// be recorded into CUDA graphs:
//
//   route    one warp per token: softmax over all router outputs in 32-bit, choice scores
//            (score + correction), groups of neighbouring outputs of which only the best
//            `keep` (by their largest choice score) stay eligible, the `top` largest choice
//            scores (ties: the lower index), weights = the chosen outputs' scores over their
//            sum (+ 1e-20).  Outputs from n_real on are identity experts: they need no
//            product.  Counts the tokens of every real expert.
//   plan     offsets of the experts' token lists and the list of row tiles (expert, first
//            row, rows) that the grouped products walk.
//   scatter  every (token, choice) pair takes a place in its expert's list.
//   product  Y[place] = act(X[token] Wg_e^T) * (X[token] Wu_e^T)  (gated, rows gathered), or
//            Y[place] = X[place] W_e^T; one CTA per (row tile, 64 features); a tile holds rows
//            of ONE expert.  Every output is one chain of fused multiply-adds over k in
//            ascending order, so a token's result depends neither on its place nor on the batch.
//   combine  out[token] = sum over its choices, in the order of the choices, of weight *
//            (the expert's output row, or the token's own input for an identity expert)
//            + the shared expert's output, in 32-bit, rounded once.
#include "common.cuh"

namespace sllm {

constexpr int MOE_TM = 32;   // rows of a tile
constexpr int MOE_TN = 64;   // features of a tile
constexpr int MOE_TK = 16;
constexpr int MOE_MAX_TOP = 32;
// router variants (bits of `flags`): scores are sigmoid(z) instead of a softmax over all outputs;
// a group's score is the sum of its two largest choice scores instead of its largest; the
// weights are the chosen scores themselves, not divided by their sum
constexpr int MOE_SIGMOID = 1, MOE_GROUP_TOP2 = 2, MOE_RAW_WEIGHTS = 4;

// One warp routes one token.  z: the token's n_total router logits; score: 2 n_total + 2 n_groups
// floats of shared memory of this warp; counts: the experts' counters (global or shared memory).
__device__ __forceinline__ void route_token(const float* __restrict__ z,
                                            const float* __restrict__ corr, float* score,
                                            int n_total, int n_real, int n_groups, int keep,
                                            int top, int lane, int* __restrict__ ids_row,
                                            float* __restrict__ weights_row, int* counts,
                                            int flags) {
    float* choice = score + n_total;   // score + correction, -inf once taken or barred
    if (flags & MOE_SIGMOID) {
        for (int e = lane; e < n_total; e += 32) {
            const float s = 1.0f / (1.0f + expf(-z[e]));
            score[e] = s;
            choice[e] = s + corr[e];
        }
    } else {
        float m = -INFINITY;
        for (int e = lane; e < n_total; e += 32) m = fmaxf(m, z[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < n_total; e += 32) {
            const float p = expf(z[e] - m);
            score[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        for (int e = lane; e < n_total; e += 32) {
            const float s = score[e] / sum;
            score[e] = s;
            choice[e] = s + corr[e];
        }
    }
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        // a group's score is its largest choice score (or, with MOE_GROUP_TOP2, the sum of its
        // two largest); the `keep` best groups (ties: the lower index) stay, every output of the
        // others is barred
        const int per = n_total / n_groups;
        float* gscore = choice + n_total;
        float* gkept = gscore + n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float best = -INFINITY, second = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float c = choice[e];
                if (c > best) {
                    second = best;
                    best = c;
                } else if (c > second) {
                    second = c;
                }
            }
            gscore[g] = ((flags & MOE_GROUP_TOP2) && per > 1) ? best + second : best;
            gkept[g] = 0.f;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int best_g = -1;
            for (int g = lane; g < n_groups; g += 32)
                if (gkept[g] == 0.f && (best_g < 0 || gscore[g] > best)) {
                    best = gscore[g];
                    best_g = g;
                }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                if (og >= 0 && (best_g < 0 || ov > best || (ov == best && og < best_g))) {
                    best = ov;
                    best_g = og;
                }
            }
            __syncwarp();
            if (lane == 0 && best_g >= 0) gkept[best_g] = 1.f;
            __syncwarp();
        }
        for (int e = lane; e < n_total; e += 32)
            if (gkept[e / per] == 0.f) choice[e] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f;
    float my_w = 0.f;
    int my_id = -1;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = -1;
        for (int e = lane; e < n_total; e += 32) {
            const float c = choice[e];
            if (c > best) {
                best = c;
                best_e = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe >= 0 && (best_e < 0 || ov > best || (ov == best && oe < best_e))) {
                best = ov;
                best_e = oe;
            }
        }
        float s = 0.f;
        if (best_e >= 0) {
            s = score[best_e];
            __syncwarp();
            if (lane == 0) choice[best_e] = -INFINITY;
            __syncwarp();
        }
        wsum += s;
        if (lane == k) {
            my_w = s;
            my_id = best_e;
        }
    }
    if (lane < top) {
        ids_row[lane] = my_id;
        weights_row[lane] = (flags & MOE_RAW_WEIGHTS) ? my_w : my_w / (wsum + 1e-20f);
        if (my_id >= 0 && my_id < n_real) atomicAdd(&counts[my_id], 1);
    }
}

// logits: float32 [N, n_total]; shared memory: warps * (2 n_total + 2 n_groups) floats.
__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ corr,
                                 const int* __restrict__ token_row, int N, int n_total,
                                 int n_real, int n_groups, int keep, int top,
                                 int* __restrict__ ids, float* __restrict__ weights,
                                 int* __restrict__ counts, int flags) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= N) return;
    if (token_row != nullptr && token_row[n] < 0) {     // a padding token goes nowhere
        for (int k = lane; k < top; k += 32) {
            ids[(int64_t)n * top + k] = -1;
            weights[(int64_t)n * top + k] = 0.f;
        }
        return;
    }
    route_token(logits + (int64_t)n * n_total, corr,
                smem + (size_t)warp * (2 * n_total + 2 * n_groups), n_total, n_real, n_groups, keep,
                top, lane, ids + (int64_t)n * top, weights + (int64_t)n * top, counts, flags);
}

// Steps of few tokens (decode): ONE CTA routes every token, counts, plans the tiles, gives every
// (token, choice) pair its place and, for the tensor-core products, copies the tokens' rows into
// the sorted order (x: bfloat16 rows of K elements, K % 8 == 0; rows_out null: no copy), where
// the general path runs a fill, three kernels and a copy.  Nothing has to be zeroed beforehand.
// Shared memory: 8 warps' routing scratch, then counts [E], offsets [E + 1], cursor [E].
constexpr int MOE_SMALL_WARPS = 8;
__global__ void __launch_bounds__(MOE_SMALL_WARPS * 32)
moe_route_small_kernel(const float* __restrict__ logits, const float* __restrict__ corr,
                       const int* __restrict__ token_row, int N, int n_total, int n_real,
                       int n_groups, int keep, int top, int* __restrict__ ids,
                       float* __restrict__ weights, int* __restrict__ meta, int max_tiles,
                       int tile_rows, int* __restrict__ pair_token, int* __restrict__ pair_place,
                       const __nv_bfloat16* __restrict__ x, int64_t ldx, int K,
                       __nv_bfloat16* __restrict__ rows_out, int flags) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int per_warp = 2 * n_total + 2 * n_groups;
    int* counts = reinterpret_cast<int*>(smem + (size_t)MOE_SMALL_WARPS * per_warp);
    int* offsets = counts + n_real;
    int* cursor = offsets + n_real + 1;
    const int n_pairs = N * top;
    for (int e = tid; e < n_real; e += blockDim.x) counts[e] = cursor[e] = 0;
    for (int p = tid; p < n_pairs; p += blockDim.x) pair_token[p] = 0;   // places nobody takes
    __syncthreads();
    for (int n = warp; n < N; n += MOE_SMALL_WARPS) {
        if (token_row != nullptr && token_row[n] < 0) {
            for (int k = lane; k < top; k += 32) {
                ids[(int64_t)n * top + k] = -1;
                weights[(int64_t)n * top + k] = 0.f;
            }
            continue;
        }
        route_token(logits + (int64_t)n * n_total, corr, smem + (size_t)warp * per_warp, n_total,
                    n_real, n_groups, keep, top, lane, ids + (int64_t)n * top,
                    weights + (int64_t)n * top, counts, flags);
    }
    __syncthreads();
    for (int e = tid; e <= n_real; e += blockDim.x) {
        int off = 0, tiles = 0;
        for (int j = 0; j < e; ++j) {
            off += counts[j];
            tiles += (counts[j] + tile_rows - 1) / tile_rows;
        }
        offsets[e] = off;
        if (e == n_real) {
            meta[0] = min(tiles, max_tiles);
            continue;
        }
        const int c = counts[e];
        for (int i = 0; i * tile_rows < c && tiles + i < max_tiles; ++i) {
            int* t = meta + 1 + 3 * (tiles + i);
            t[0] = e;
            t[1] = off + i * tile_rows;
            t[2] = min(tile_rows, c - i * tile_rows);
        }
    }
    __syncthreads();
    for (int i = tid; i < n_pairs; i += blockDim.x) {
        const int e = ids[i];
        int place = -1;
        if (e >= 0 && e < n_real) {
            place = offsets[e] + atomicAdd(&cursor[e], 1);
            pair_token[place] = i / top;
        }
        pair_place[i] = place;
    }
    if (rows_out == nullptr) return;
    __syncthreads();
    const int units = K / 8;
    for (int i = tid; i < n_pairs * units; i += blockDim.x) {
        const int p = i / units, u = i - p * units;
        reinterpret_cast<uint4*>(rows_out + (int64_t)p * K)[u] =
            reinterpret_cast<const uint4*>(x + (int64_t)pair_token[p] * ldx)[u];
    }
}

// One block.  counts [E] -> offsets [E + 1], cursor [E] = 0, the tile list and its length.
// meta: int32 [1 + 3 * max_tiles]: n_tiles, then (expert, first row, rows) per tile of up to
// tile_rows rows (what the product kernel that follows takes: MOE_TM here, 128 on tcgen05).
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                int* __restrict__ cursor, int* __restrict__ meta, int max_tiles,
                                int tile_rows) {
    pdl_wait();
    pdl_trigger();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) {
        int off = 0, tiles = 0;
        for (int j = 0; j < e; ++j) {
            off += counts[j];
            tiles += (counts[j] + tile_rows - 1) / tile_rows;
        }
        offsets[e] = off;
        if (e == E) {
            meta[0] = min(tiles, max_tiles);
            continue;
        }
        cursor[e] = 0;
        const int c = counts[e];
        for (int i = 0; i * tile_rows < c && tiles + i < max_tiles; ++i) {
            int* t = meta + 1 + 3 * (tiles + i);
            t[0] = e;
            t[1] = off + i * tile_rows;
            t[2] = min(tile_rows, c - i * tile_rows);
        }
    }
}

// pair_token [P]: the token of each place; pair_place [N * top]: the place of each (token,
// choice), -1 for identity experts and padding.
__global__ void moe_scatter_kernel(const int* __restrict__ ids, int n_pairs, int top, int n_real,
                                   const int* __restrict__ offsets, int* __restrict__ cursor,
                                   int* __restrict__ pair_token, int* __restrict__ pair_place) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int e = ids[i];
    int place = -1;
    if (e >= 0 && e < n_real) {
        place = offsets[e] + atomicAdd(&cursor[e], 1);
        pair_token[place] = i / top;
    }
    pair_place[i] = place;
}

// grid (ceil(F / MOE_TN), max_tiles).  MODE 1 (gated): W is [E, 2 F, K] (gate rows, then up
// rows), Y[place, f] = silu(x . gate_f) * (x . up_f) with x = X[pair_token[place]].  MODE 2
// (an expert without a gate): W is [E, F, K], Y[place, f] = relu(x . w_f)^2 with the same
// gathered x.  MODE 0: W is [E, F, K], Y[place, f] = X[place] . w_f.
template <typename TIn, typename TOut, int MODE>
__global__ void __launch_bounds__(256)
moe_product_kernel(const TIn* __restrict__ X, int64_t ldx, const TIn* __restrict__ W,
                   TOut* __restrict__ Y, int64_t ldy, const int* __restrict__ meta,
                   const int* __restrict__ pair_token, int F, int K) {
    pdl_wait();
    pdl_trigger();
    constexpr bool GATED = MODE == 1, GATHER = MODE != 0;
    if ((int)blockIdx.y >= meta[0]) return;
    const int* tile = meta + 1 + 3 * blockIdx.y;
    const int expert = tile[0], row0 = tile[1], rows = tile[2];
    __shared__ float As[MOE_TK][MOE_TM + 4];
    __shared__ float Bs[GATED ? 2 : 1][MOE_TK][MOE_TN + 4];
    __shared__ int src_row[MOE_TM];
    const int tid = threadIdx.x;
    if (tid < MOE_TM) src_row[tid] = tid < rows ? (GATHER ? pair_token[row0 + tid] : row0 + tid) : -1;
    __syncthreads();
    const int f0 = blockIdx.x * MOE_TN;
    const TIn* We = W + (int64_t)expert * (GATED ? 2 : 1) * F * K;
    const int ty = tid >> 4, tx = tid & 15;       // 2 rows x 4 features per thread
    float acc[GATED ? 2 : 1][2][4];
#pragma unroll
    for (int s = 0; s < (GATED ? 2 : 1); ++s)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[s][i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_TK) {
        // A: 32 rows x 16 k = 512 values, two per thread; B: 64 x 16 (x 2), four per thread
        for (int i = tid; i < MOE_TM * MOE_TK; i += 256) {
            const int r = i / MOE_TK, k = i - r * MOE_TK;
            const int src = src_row[r];
            As[k][r] = (src >= 0 && k0 + k < K) ? to_float(X[(int64_t)src * ldx + k0 + k]) : 0.f;
        }
        for (int i = tid; i < MOE_TN * MOE_TK; i += 256) {
            const int f = i / MOE_TK, k = i - f * MOE_TK;
            const bool ok = f0 + f < F && k0 + k < K;
            Bs[0][k][f] = ok ? to_float(We[(int64_t)(f0 + f) * K + k0 + k]) : 0.f;
            if (GATED) Bs[1][k][f] = ok ? to_float(We[(int64_t)(F + f0 + f) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; ++kk) {
            float a[2], b[GATED ? 2 : 1][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) a[i] = As[kk][ty * 2 + i];
#pragma unroll
            for (int s = 0; s < (GATED ? 2 : 1); ++s)
#pragma unroll
                for (int j = 0; j < 4; ++j) b[s][j] = Bs[s][kk][tx * 4 + j];
#pragma unroll
            for (int s = 0; s < (GATED ? 2 : 1); ++s)
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[s][i][j] = fmaf(a[i], b[s][j], acc[s][i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty * 2 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int f = f0 + tx * 4 + j;
            if (f >= F) continue;
            float y = acc[0][i][j];
            if (GATED) {
                const float g = y, u = acc[GATED ? 1 : 0][i][j];
                y = g / (1.0f + expf(-g)) * u;
            } else if (MODE == 2) {
                y = y > 0.f ? y * y : 0.f;
            }
            Y[(int64_t)(row0 + r) * ldy + f] = from_float<TOut>(y);
        }
    }
}

// One block per token.  y: float32 [P, d]; x: the feed-forward's own input [N, d]; shared (may
// be null): the shared expert's output [N, d].
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const T* __restrict__ x,
                                   const T* __restrict__ shared, const int* __restrict__ ids,
                                   const float* __restrict__ weights,
                                   const int* __restrict__ pair_place, int top, int n_real, int d,
                                   T* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int id = ids[n * top + k];
            if (id < 0) continue;
            const float w = weights[n * top + k];
            const float v = id >= n_real ? to_float(x[n * d + e])
                                         : y[(int64_t)pair_place[n * top + k] * d + e];
            acc = fmaf(w, v, acc);
        }
        if (shared != nullptr) acc += to_float(shared[n * d + e]);
        out[n * d + e] = from_float<T>(acc);
    }
}

// The same with four features per thread (d % 4 == 0, 16-byte reads of y).
template <typename T> struct Quad;
template <> struct Quad<float> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Quad<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
        v[0] = __low2float(h[0]); v[1] = __high2float(h[0]);
        v[2] = __low2float(h[1]); v[3] = __high2float(h[1]);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        uint2 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
        h[0] = __floats2bfloat162_rn(v[0], v[1]);
        h[1] = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

template <typename T>
__global__ void moe_combine_vec_kernel(const float* __restrict__ y, const T* __restrict__ x,
                                       const T* __restrict__ shared, const int* __restrict__ ids,
                                       const float* __restrict__ weights,
                                       const int* __restrict__ pair_place, int top, int n_real,
                                       int d, T* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    for (int e = 4 * threadIdx.x; e < d; e += 4 * blockDim.x) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
        for (int k = 0; k < top; ++k) {
            const int id = ids[n * top + k];
            if (id < 0) continue;
            const float w = weights[n * top + k];
            if (id >= n_real) Quad<T>::load(x + n * d + e, v);
            else Quad<float>::load(y + (int64_t)pair_place[n * top + k] * d + e, v);
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[q] = fmaf(w, v[q], acc[q]);
        }
        if (shared != nullptr) {
            Quad<T>::load(shared + n * d + e, v);
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[q] += v[q];
        }
        Quad<T>::store(out + n * d + e, acc);
    }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_moe_tile_rows() { return MOE_TM; }

// work: int32, zero-filled by the caller: counts [E], then offsets [E + 1], cursor [E],
// meta [1 + 3 * max_tiles].
SLLM_EXPORT int sllm_moe_route(const float* logits, const float* corr, const int* token_row,
                               int n_tokens, int n_total, int n_real, int n_groups, int keep,
                               int top, int* ids, float* weights, int* work, int max_tiles,
                               int tile_rows, int* pair_token, int* pair_place, int flags,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_total <= 0 || n_real < 0 || n_real > n_total || top < 1 || top > MOE_MAX_TOP ||
        top > n_total || n_groups < 1 || n_total % n_groups || keep < 1 || keep > n_groups ||
        n_total > 4096 || tile_rows < 1)
        return (int)cudaErrorInvalidValue;
    const int warps = 4;
    int* counts = work;
    int* offsets = counts + n_real;
    int* cursor = offsets + n_real + 1;
    int* meta = cursor + n_real;
    cudaError_t err = sllm_launch_pdl(moe_route_kernel, dim3((n_tokens + warps - 1) / warps),
                                      dim3(32 * warps),
                                      (size_t)warps * (2 * n_total + 2 * n_groups) * sizeof(float),
                                      stream, logits, corr, token_row, n_tokens, n_total, n_real,
                                      n_groups, keep, top, ids, weights, counts, flags);
    if (err != cudaSuccess) return (int)err;
    if (n_real == 0) return 0;
    err = sllm_launch_pdl(moe_plan_kernel, dim3(1), dim3(256), 0, stream, (const int*)counts,
                          n_real, offsets, cursor, meta, max_tiles, tile_rows);
    if (err != cudaSuccess) return (int)err;
    const int n_pairs = n_tokens * top;
    return (int)sllm_launch_pdl(moe_scatter_kernel, dim3((n_pairs + 255) / 256), dim3(256), 0,
                                stream, (const int*)ids, n_pairs, top, n_real,
                                (const int*)offsets, cursor, pair_token, pair_place);
}

// Shared memory the one-CTA router needs for these sizes (the caller checks it against 48 KB).
SLLM_EXPORT int sllm_moe_route_small_smem(int n_total, int n_real, int n_groups) {
    return (MOE_SMALL_WARPS * (2 * n_total + 2 * n_groups) + 3 * n_real + 1) * 4;
}

// The router, the plan, the scatter and the copy of the rows in one launch, for steps of few
// tokens.  meta: int32 [1 + 3 * max_tiles]; x / rows_out (bfloat16, may be null): see the kernel.
SLLM_EXPORT int sllm_moe_route_small(const float* logits, const float* corr, const int* token_row,
                                     int n_tokens, int n_total, int n_real, int n_groups, int keep,
                                     int top, int* ids, float* weights, int* meta, int max_tiles,
                                     int tile_rows, int* pair_token, int* pair_place,
                                     const void* x, int64_t ldx, int K, void* rows_out, int flags,
                                     cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_total <= 0 || n_real < 0 || n_real > n_total || top < 1 || top > MOE_MAX_TOP ||
        top > n_total || n_groups < 1 || n_total % n_groups || keep < 1 || keep > n_groups ||
        tile_rows < 1 || max_tiles < 1)
        return (int)cudaErrorInvalidValue;
    if (rows_out != nullptr &&
        (x == nullptr || K <= 0 || (K % 8) || (ldx % 8) || (((uintptr_t)x | (uintptr_t)rows_out) & 15)))
        return (int)cudaErrorInvalidValue;
    const int smem = sllm_moe_route_small_smem(n_total, n_real, n_groups);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return (int)sllm_launch_pdl(moe_route_small_kernel, dim3(1), dim3(MOE_SMALL_WARPS * 32),
                                (size_t)smem, stream, logits, corr, token_row, n_tokens, n_total,
                                n_real, n_groups, keep, top, ids, weights, meta, max_tiles,
                                tile_rows, pair_token, pair_place, (const __nv_bfloat16*)x, ldx, K,
                                (__nv_bfloat16*)rows_out, flags);
}

// dtype: 0 = float32 operands, 1 = bfloat16 operands.  gated 1 (silu(gate) * up) and 2 (squared
// relu of one matrix): rows gathered through pair_token, Y has the operands' dtype; 0: Y is
// float32.
SLLM_EXPORT int sllm_moe_product(const void* X, int64_t ldx, const void* W, void* Y, int64_t ldy,
                                 const int* meta, const int* pair_token, int F, int K,
                                 int max_tiles, int gated, int dtype, cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    if (F <= 0 || K <= 0 || max_tiles > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((F + MOE_TN - 1) / MOE_TN, max_tiles);
    typedef __nv_bfloat16 bf16;
    cudaError_t err;
    if (gated < 0 || gated > 2) return (int)cudaErrorInvalidValue;
    if (dtype == 0 && gated == 1)
        err = sllm_launch_pdl(moe_product_kernel<float, float, 1>, grid, dim3(256), 0, stream,
                              (const float*)X, ldx, (const float*)W, (float*)Y, ldy, meta,
                              pair_token, F, K);
    else if (dtype == 0 && gated == 2)
        err = sllm_launch_pdl(moe_product_kernel<float, float, 2>, grid, dim3(256), 0, stream,
                              (const float*)X, ldx, (const float*)W, (float*)Y, ldy, meta,
                              pair_token, F, K);
    else if (dtype == 0)
        err = sllm_launch_pdl(moe_product_kernel<float, float, 0>, grid, dim3(256), 0, stream,
                              (const float*)X, ldx, (const float*)W, (float*)Y, ldy, meta,
                              pair_token, F, K);
    else if (dtype == 1 && gated == 1)
        err = sllm_launch_pdl(moe_product_kernel<bf16, bf16, 1>, grid, dim3(256), 0, stream,
                              (const bf16*)X, ldx, (const bf16*)W, (bf16*)Y, ldy, meta, pair_token,
                              F, K);
    else if (dtype == 1 && gated == 2)
        err = sllm_launch_pdl(moe_product_kernel<bf16, bf16, 2>, grid, dim3(256), 0, stream,
                              (const bf16*)X, ldx, (const bf16*)W, (bf16*)Y, ldy, meta, pair_token,
                              F, K);
    else if (dtype == 1)
        err = sllm_launch_pdl(moe_product_kernel<bf16, float, 0>, grid, dim3(256), 0, stream,
                              (const bf16*)X, ldx, (const bf16*)W, (float*)Y, ldy, meta,
                              pair_token, F, K);
    else
        return (int)cudaErrorInvalidValue;
    return (int)err;
}

SLLM_EXPORT int sllm_moe_combine(const float* y, const void* x, const void* shared, const int* ids,
                                 const float* weights, const int* pair_place, int n_tokens,
                                 int top, int n_real, int d, void* out, int dtype,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0) return (int)cudaErrorInvalidValue;
    typedef __nv_bfloat16 bf16;
    if (d % 4 == 0 && !(((uintptr_t)y | (uintptr_t)x | (uintptr_t)shared | (uintptr_t)out) & 15)) {
        int vt = 32;
        while (vt < 256 && vt * 4 < d) vt <<= 1;
        if (dtype == 0)
            return (int)sllm_launch_pdl(moe_combine_vec_kernel<float>, dim3(n_tokens), dim3(vt), 0,
                                        stream, y, (const float*)x, (const float*)shared, ids,
                                        weights, pair_place, top, n_real, d, (float*)out);
        if (dtype == 1)
            return (int)sllm_launch_pdl(moe_combine_vec_kernel<bf16>, dim3(n_tokens), dim3(vt), 0,
                                        stream, y, (const bf16*)x, (const bf16*)shared, ids,
                                        weights, pair_place, top, n_real, d, (bf16*)out);
        return (int)cudaErrorInvalidValue;
    }
    const int threads = d >= 256 ? 256 : 128;
    if (dtype == 0)
        return (int)sllm_launch_pdl(moe_combine_kernel<float>, dim3(n_tokens), dim3(threads), 0,
                                    stream, y, (const float*)x, (const float*)shared, ids, weights,
                                    pair_place, top, n_real, d, (float*)out);
    if (dtype == 1)
        return (int)sllm_launch_pdl(moe_combine_kernel<bf16>, dim3(n_tokens), dim3(threads), 0,
                                    stream, y, (const bf16*)x, (const bf16*)shared, ids, weights,
                                    pair_place, top, n_real, d, (bf16*)out);
    return (int)cudaErrorInvalidValue;
}
