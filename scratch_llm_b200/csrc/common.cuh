// Shared device helpers for the engine's kernels (sm_100a).
//
// Every launcher is an extern "C" function that takes raw device pointers, sizes and the
// CUDA stream to launch on, allocates nothing, and returns a cudaError_t as int (0 = ok).
// Launchers check sizes they cannot handle and return cudaErrorInvalidValue instead of
// computing a wrong result; the Python binding turns any non-zero code into an exception.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SLLM_EXPORT extern "C" __attribute__((visibility("default")))

#define SLLM_LAUNCH_CHECK()                          \
    do {                                             \
        cudaError_t e__ = cudaGetLastError();        \
        if (e__ != cudaSuccess) return (int)e__;     \
    } while (0)

namespace sllm {

// Programmatic dependent launch.  pdl_trigger() lets the next kernel in the stream start to be
// scheduled while this one still runs; it only takes effect if that kernel was launched with
// the programmatic-stream-serialization attribute, and such a kernel must call pdl_wait()
// before it reads or writes anything an earlier kernel may touch (weights, which nothing
// writes, may be read before).  pdl_wait() returns once all earlier kernels have completed
// and their writes are visible; without the launch attribute it returns at once.
// Every kernel here calls pdl_wait() FIRST and pdl_trigger() right after it: a trigger before
// the wait would let the whole chain of later kernels pile up on the SMs, each parked in its
// wait and holding registers and shared memory that the running kernel needs (measured: the
// decode step became 60 % slower).  This way at most one kernel is parked ahead.
__device__ __forceinline__ void pdl_trigger() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

}  // namespace sllm

// Launch with programmatic stream serialization: the kernel may be scheduled while the previous
// kernel of the stream drains, and must call sllm::pdl_wait() before touching that kernel's data.
template <typename... KArgs, typename... Args>
static inline cudaError_t sllm_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                          size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

namespace sllm {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// 16 bytes at a time: 4 floats or 8 bfloat16, as floats.
template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        const uint4 r = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __low2float(h[i]);
            v[2 * i + 1] = __high2float(h[i]);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        uint4 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = r;
    }
};

// The activation on the gate of a gated feed-forward, act(gate) * up: act = 1 is silu,
// act = 2 the tanh form of gelu, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
__device__ __forceinline__ float gate_activation(float z, int act) {
    if (act == 2) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.0f + expf(-z));
}
// The same with the hardware's approximations (relative error below bfloat16's rounding), for
// epilogues that sit on a tensor-core kernel's critical path.
__device__ __forceinline__ float gate_activation_fast(float z, int act) {
    if (act == 2) {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        return 0.5f * z * (1.0f + t);
    }
    return z / (1.0f + __expf(-z));
}

// What a gated feed-forward multiplies its down matrix with, from a gate and an up value.
// act 1, 2: act(gate) * up as above.  act 3, with p0 = a limit and p1 = a slope: the gate is
// clamped from above and the up value on both sides, g = min(gate, p0), u = clamp(up, -p0, p0),
// and the product is g * sigmoid(p1 * g) * (u + 1).
__device__ __forceinline__ float gated_product(float gate, float up, int act, float p0, float p1) {
    if (act == 3) {
        const float g = fminf(gate, p0), u = fminf(fmaxf(up, -p0), p0);
        return g / (1.0f + expf(-p1 * g)) * (u + 1.0f);
    }
    return gate_activation(gate, act) * up;
}
__device__ __forceinline__ float gated_product_fast(float gate, float up, int act, float p0,
                                                    float p1) {
    if (act == 3) {
        const float g = fminf(gate, p0), u = fminf(fmaxf(up, -p0), p0);
        return g / (1.0f + __expf(-p1 * g)) * (u + 1.0f);
    }
    return gate_activation_fast(gate, act) * up;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33
// floats of shared memory.  The order of the additions depends only on blockDim.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace sllm
