// Shared helpers of the sm_100a kernels: element conversion, reductions, the C ABI's error reporting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FERRIS_API extern "C" __attribute__((visibility("default")))

// Error codes of the C ABI. 0 = ok; > 0 = a cudaError_t; < 0 = the launcher refused its arguments
// (ferris_last_error() gives the text).
#define FERRIS_OK 0
#define FERRIS_BAD_ARGUMENT (-1)
#define FERRIS_TIMEOUT (-2)

// Data types of the C ABI.
#define FERRIS_F32 0
#define FERRIS_BF16 1

void ferris_set_error(const char* fmt, ...);

#define FERRIS_REFUSE(...)            \
    do {                              \
        ferris_set_error(__VA_ARGS__); \
        return FERRIS_BAD_ARGUMENT;   \
    } while (0)

#define FERRIS_LAUNCH_CHECK()                          \
    do {                                               \
        cudaError_t e_ = cudaGetLastError();           \
        if (e_ != cudaSuccess) {                       \
            ferris_set_error("%s", cudaGetErrorString(e_)); \
            return (int)e_;                            \
        }                                              \
        return FERRIS_OK;                              \
    } while (0)

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched through ferris_launch may begin while the kernel
// before it in the stream is still draining.  Its set-up (barriers, tensor memory, descriptor
// prefetch) overlaps that tail; pdl_wait() then blocks until the earlier kernel has completed and its
// writes are visible, and must come before the first access to global memory.
// pdl_launch_dependents() lets the NEXT kernel start its own set-up early; it takes effect once every
// CTA of this grid has called it (or exited), so CTAs that are not resident yet are never starved.
// Launched without the attribute (FERRIS_PDL=0), both are no-ops.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool ferris_pdl_enabled();

template <typename Kernel, typename... Args>
inline cudaError_t ferris_launch(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ferris_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// The same with the CTAs of each (x, y) grouped along z into clusters of `cluster_z`.
template <typename Kernel, typename... Args>
inline cudaError_t ferris_launch_cluster(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                         unsigned cluster_z, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = cluster_z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ferris_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ bf16 from_float<bf16>(float v) {
    return __float2bfloat16_rn(v);
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

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    if (warp == 0) {
        float w = lane < nwarps ? scratch[lane] : 0.0f;
        w = warp_sum(w);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    float r = scratch[32];
    __syncthreads();
    return r;
}
