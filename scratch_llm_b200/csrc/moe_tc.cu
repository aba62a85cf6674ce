// The grouped products of a routed feed-forward in bfloat16 on the 5th-generation tensor cores
// (tcgen05): the single-SM product of gemm_tcgen05.cu (TMA with 128-byte swizzle -> a ring of
// four 48 KB stages -> tcgen05.mma, M = 128, N = 256, accumulator double-buffered in tensor
// memory -> tcgen05.ld epilogue; warp 0 produces, warp 1 issues, warps 2-5 drain; persistent
// CTAs), walking a TILE LIST that the router's plan kernel left on the device instead of a
// regular grid of tiles:
//
//   meta = [n_tiles, (expert, first row, rows) x n_tiles]: a tile is up to 128 rows of ONE
//   expert in the list of (token, choice) pairs sorted by expert.
//
// A tile's A operand is 128 rows of the sorted activations from its first row on (what lies
// beyond its `rows` belongs to the next expert, or is the zero fill beyond the matrix: those
// accumulator rows are never stored); its B operand is the expert's rows of the stacked weights
// [experts * rows per expert, K].  GATED: the expert's matrix is [gate rows; up rows], a tile
// covers 128 features (128 gate + 128 up accumulator columns) and the epilogue stores
// silu(gate) * up in bfloat16; else a tile covers 256 output features and is stored in 32-bit.
// Nothing is read on the host: the number of tiles is read from `meta` by every role, and the
// launch has a fixed grid, so the kernel can be recorded into CUDA graphs.
//
// sllm_moe_gather_rows copies the tokens' rows into the sorted order first (16-byte accesses).
//
// Every mbarrier wait is bounded (tc_common.cuh): a wait that gives up records its code in this
// library's error word, the CTA reaches its end and frees its tensor memory.
#include "tc_common.cuh"

namespace sllm {

constexpr int TM = 128, TN = 256, TK = 64, STAGES = 4;
constexpr int A_BYTES = TM * TK * 2, B_BYTES = TN * TK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TC_THREADS = 192;
constexpr size_t TC_SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

__device__ __forceinline__ void store_row32(bf16* dst, const float (&o)[32], int n_valid,
                                            bool aligned) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (aligned && n_valid >= 8 * (i + 1)) {
            uint4 q;
            q.x = pack2(o[8 * i + 0], o[8 * i + 1]);
            q.y = pack2(o[8 * i + 2], o[8 * i + 3]);
            q.z = pack2(o[8 * i + 4], o[8 * i + 5]);
            q.w = pack2(o[8 * i + 6], o[8 * i + 7]);
            reinterpret_cast<uint4*>(dst)[i] = q;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (8 * i + j < n_valid) dst[8 * i + j] = __float2bfloat16_rn(o[8 * i + j]);
        }
    }
}
__device__ __forceinline__ void store_row32(float* dst, const float (&o)[32], int n_valid,
                                            bool aligned) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (aligned && n_valid >= 4 * (i + 1)) {
            reinterpret_cast<float4*>(dst)[i] =
                make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (4 * i + j < n_valid) dst[4 * i + j] = o[4 * i + j];
        }
    }
}

// n_out: output features per expert (GATED: the gated size F, W holds 2 F rows per expert).
// Tiles are walked band by band (tile_coords): a band is MOE_BAND neighbouring row tiles through
// all feature blocks, row tiles fastest (so that an expert's row tiles, which share its weights,
// run side by side).  A band's activations (MOE_BAND x 128 rows) stay in L2 while the weights
// stream past once; without bands a step of many thousand rows re-reads all its activations
// from memory for every feature block.  Up to MOE_BAND row tiles: one band.
// SQRELU (not gated): the stored value is relu(y)^2, an expert without a gate.
constexpr int MOE_BAND = 16;
__device__ __forceinline__ void tile_coords(int tile, int n_row_tiles, int tiles_n, int& row_tile,
                                            int& n_blk) {
    const int band_tiles = MOE_BAND * tiles_n;
    const int band = tile / band_tiles;
    const int in_band = tile - band * band_tiles;
    const int rows_here = min(MOE_BAND, n_row_tiles - band * MOE_BAND);
    n_blk = in_band / rows_here;
    row_tile = band * MOE_BAND + in_band - n_blk * rows_here;
}

template <bool GATED, typename TOut, bool SQRELU = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
moe_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
              TOut* __restrict__ Y, const int* __restrict__ meta, int n_out, int K, int64_t ldy,
              int tiles_n, int max_tiles) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        ((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* a_stage = smem;                          // STAGES x 16 KB
    unsigned char* b_stage = smem + STAGES * A_BYTES;       // STAGES x 32 KB
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;     // [2]: the MMA warp has finished a tile
    uint64_t* acc_empty = acc_full + 2;      // [2]: the four epilogue warps have drained it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + TK - 1) / TK;
    int n_row_tiles = meta[0];
    if (n_row_tiles > max_tiles) n_row_tiles = max_tiles;
    if (n_row_tiles < 0) n_row_tiles = 0;
    const int total_tiles = n_row_tiles * tiles_n;
    const int rows_per_expert = GATED ? 2 * n_out : n_out;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int row_tile, n_blk;
                tile_coords(tile, n_row_tiles, tiles_n, row_tile, n_blk);
                const int* t = meta + 1 + 3 * row_tile;
                const int expert = t[0], m0 = t[1];
                const int w_base = expert * rows_per_expert;
                const int w_row0 = w_base + (GATED ? n_blk * 128 : n_blk * TN);
                const int w_row1 = GATED ? w_base + n_out + n_blk * 128 : w_row0 + 128;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, 1);
                    if (!ok) break;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(a_stage + s * A_BYTES, &map_x, &full[s], kb * TK, m0);
                    tma_load_2d(b_stage + s * B_BYTES, &map_w, &full[s], kb * TK, w_row0);
                    tma_load_2d(b_stage + s * B_BYTES + B_BYTES / 2, &map_w, &full[s], kb * TK,
                                w_row1);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) |
                                   ((uint32_t)(TM >> 4) << 24);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
                const uint32_t buf = local & 1;
                ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * TN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = make_smem_desc(smem_u32(a_stage + s * A_BYTES));
                    const uint64_t db = make_smem_desc(smem_u32(b_stage + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < TK / 16; ++k)
                        umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit(&empty[s]);
                }
                umma_commit(&acc_full[buf]);
            }
        }
    } else {
        const int quad = warp & 3;        // the 32 tensor-memory lanes this warp may read
        uint32_t local = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
            const uint32_t buf = local & 1;
            int row_tile, n_blk;
            tile_coords(tile, n_row_tiles, tiles_n, row_tile, n_blk);
            const int* t = meta + 1 + 3 * row_tile;
            const int m0 = t[1], rows = t[2];
            const int r = quad * 32 + lane;
            if (!mbar_wait(&acc_full[buf], (local >> 1) & 1, 3)) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + buf * TN + ((uint32_t)(quad * 32) << 16);
            const bool aligned = (ldy % (16 / (int)sizeof(TOut))) == 0;
            TOut* dst = Y + (int64_t)(m0 + r) * ldy;
            if (!GATED) {
                const int n0 = n_blk * TN;
#pragma unroll 1
                for (int c = 0; c < TN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(lane_addr + c * 32, v);
                    tmem_ld_wait();
                    const int col = n0 + c * 32;
                    if (r < rows && col < n_out) {
                        float o[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            o[i] = __uint_as_float(v[i]);
                            if (SQRELU) o[i] = o[i] > 0.f ? o[i] * o[i] : 0.f;
                        }
                        store_row32(dst + col, o, n_out - col, aligned);
                    }
                }
            } else {
                const int f0 = n_blk * 128;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t gv[32], uv[32];
                    tmem_ld32(lane_addr + c * 32, gv);
                    tmem_ld32(lane_addr + 128 + c * 32, uv);
                    tmem_ld_wait();
                    const int col = f0 + c * 32;
                    if (r < rows && col < n_out) {
                        float o[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float g = __uint_as_float(gv[i]);
                            o[i] = g / (1.0f + __expf(-g)) * __uint_as_float(uv[i]);
                        }
                        store_row32(dst + col, o, n_out - col, aligned);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n"
                     ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// out[p, :] = x[pair_token[p], :] in units of 16 bytes (K % 8 == 0).
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ x, int64_t ldx,
                                       const int* __restrict__ pair_token, int64_t n_units,
                                       int units_per_row, bf16* __restrict__ out) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_units;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t p = i / units_per_row;
        const int u = (int)(i - p * units_per_row);
        reinterpret_cast<uint4*>(out + p * units_per_row * 8)[u] =
            reinterpret_cast<const uint4*>(x + (int64_t)pair_token[p] * ldx)[u];
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld, boxes of 128 rows x 64 columns, 128-byte
// swizzle; what a box covers beyond the matrix reads as zeros.
static bool make_map(CUtensorMap* map, const void* base, int64_t rows, int K, int64_t ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TK, 128u};
    cuuint32_t elem[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_moe_tc_tile_rows() { return TM; }

// The first error a bounded wait recorded since the last call (0 = none).  Synchronises.
SLLM_EXPORT int sllm_gemm_tc_error() {
    int code = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&code, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (code) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    return code;
}

SLLM_EXPORT int sllm_moe_gather_rows(const void* x, int64_t ldx, const int* pair_token,
                                     int n_pairs, int K, void* out, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (K <= 0 || (K % 8) || (ldx % 8) || (((uintptr_t)x | (uintptr_t)out) & 15))
        return (int)cudaErrorInvalidValue;
    const int64_t units = (int64_t)n_pairs * (K / 8);
    int64_t blocks = (units + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    moe_gather_rows_kernel<<<(int)blocks, 256, 0, stream>>>((const bf16*)x, ldx, pair_token, units,
                                                            K / 8, (bf16*)out);
    SLLM_LAUNCH_CHECK();
    return 0;
}

// X: bfloat16 [n_rows, K] (rows in the sorted order), W: bfloat16 [experts * rows per expert, K]
// contiguous, Y: [n_rows, n_out] bfloat16 (gated 1: silu(gate) * up of [gate rows; up rows];
// gated 2: relu(x w)^2 of one matrix) or float32 (gated 0).  meta: the tile list of tiles of
// 128 rows; max_tiles bounds its length.
SLLM_EXPORT int sllm_moe_tc_product(const void* X, int64_t n_rows, const void* W, int n_experts,
                                    void* Y, const int* meta, int n_out, int K, int max_tiles,
                                    int gated, cudaStream_t stream) {
    if (max_tiles <= 0 || n_rows <= 0) return 0;
    if (n_out <= 0 || K <= 0 || (K % 8) || n_experts <= 0 ||
        (((uintptr_t)X | (uintptr_t)W | (uintptr_t)Y) & 15))
        return (int)cudaErrorInvalidValue;
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return (int)cudaErrorUnknown;
    }
    if (gated < 0 || gated > 2) return (int)cudaErrorInvalidValue;
    const int64_t w_rows = (int64_t)n_experts * (gated == 1 ? 2 : 1) * n_out;
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, X, n_rows, K, K) || !make_map(&map_w, W, w_rows, K, K))
        return (int)cudaErrorNotSupported;
    const int tiles_n = gated == 1 ? (n_out + 127) / 128 : (n_out + TN - 1) / TN;
    const int64_t total = (int64_t)max_tiles * tiles_n;
    if (total > 0x7fffffff) return (int)cudaErrorInvalidValue;
    dim3 grid((unsigned)(total < n_sm ? total : n_sm));
    cudaError_t e;
    if (gated == 2) {
        e = cudaFuncSetAttribute(moe_tc_kernel<false, bf16, true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
        if (e != cudaSuccess) return (int)e;
        moe_tc_kernel<false, bf16, true><<<grid, TC_THREADS, TC_SMEM, stream>>>(
            map_x, map_w, (bf16*)Y, meta, n_out, K, (int64_t)n_out, tiles_n, max_tiles);
    } else if (gated) {
        e = cudaFuncSetAttribute(moe_tc_kernel<true, bf16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
        if (e != cudaSuccess) return (int)e;
        moe_tc_kernel<true, bf16><<<grid, TC_THREADS, TC_SMEM, stream>>>(
            map_x, map_w, (bf16*)Y, meta, n_out, K, (int64_t)n_out, tiles_n, max_tiles);
    } else {
        e = cudaFuncSetAttribute(moe_tc_kernel<false, float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
        if (e != cudaSuccess) return (int)e;
        moe_tc_kernel<false, float><<<grid, TC_THREADS, TC_SMEM, stream>>>(
            map_x, map_w, (float*)Y, meta, n_out, K, (int64_t)n_out, tiles_n, max_tiles);
    }
    SLLM_LAUNCH_CHECK();
    return 0;
}
