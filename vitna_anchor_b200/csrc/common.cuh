// Shared device helpers for the sm_100a kernels of this engine.
//
// Storage types are float and __nv_bfloat16; arithmetic is always float32.
// A bfloat16 value is widened exactly (its 16 bits are the high half of a
// float32), as the reference widens stored weights (engine/src/ops.c:25-30).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define VK_API extern "C" __attribute__((visibility("default")))

// Status codes returned by every launcher.  0 is success; positive values are
// cudaError_t of the launch; negative values are refusals decided on the host
// before anything was launched.
#define VK_OK 0
#define VK_BAD_SHAPE (-1)      // a size this kernel does not take
#define VK_BAD_ALIGNMENT (-2)  // a pointer or stride that is not aligned as needed
#define VK_TOO_LARGE (-3)      // beyond a stated maximum

namespace vk {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds at least 32 floats and may be reused after the call returns.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    r = warp_sum(r);
    return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// Sixteen bytes of T as floats: 4 float32 or 8 bfloat16 (widened exactly).  p must be 16-byte aligned.
template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void load16(const T* p, float* f);
template <> __device__ __forceinline__ void load16<float>(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

inline int launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch.  A kernel launched with launch_dependent() may start while the kernel before it
// in the stream is still running; what it does before dependency_wait() must touch only memory that the kernel
// before it does not write: weights, tables, the step's metadata, and (decode attention) the keys and values of
// earlier steps.  Every kernel calls let_dependents_start() after its own dependency_wait(), so when a prologue
// runs, everything but the kernel directly before it has finished.  dependency_wait() returns when the kernel before
// it has finished and its writes are visible; let_dependents_start() allows the kernel after this one to begin
// its own prologue.  Calling them in a kernel launched the ordinary way does nothing.
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_dependents_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// An ordinary launch through the same interface (for kernels measured to run better without the overlap).
template <typename... KArgs, typename... Args>
inline int launch_plain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
inline int launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    static const bool plain = getenv("VITNA_NO_DEPENDENT_LAUNCH") != nullptr;      // for measurements: ordinary launches
    cfg.attrs = attr;
    cfg.numAttrs = plain ? 0 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace vk
