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

// Allow `fn` (a kernel) `bytes` of dynamic shared memory on the current device; the driver is asked only when the
// size grows.  Returns FERRIS_OK or a cudaError_t (text in ferris_last_error()).
int ferris_allow_dynamic_smem(const void* fn, size_t bytes);

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
// What a kernel reads after the wait from the launch before it must not come through a `const T* __restrict__`
// parameter: the compiler takes such memory for unchanging during the kernel, may load it through the non-coherent
// path and may move the load above the wait (the "memory" clobber does not hold back a load it believes invariant),
// and then reads what the buffer held a launch or a step ago.  Only weights, tables and the step's metadata are
// declared that way; activations, caches, logits and partial results are plain pointers.
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

// ---------------------------------------------------------------------------------------------
// Timeline of a step as it runs (compiled in with -DFERRIS_TIMELINE only; otherwise the hooks are
// empty).  Every instrumented kernel records, per launch, the earliest entry of a CTA, the earliest
// moment a CTA passed its programmatic-launch wait and the latest end of a CTA, in nanoseconds of
// %globaltimer.  Launches take slots in the order in which they complete.  buf[0] = next slot,
// buf[1] = slots, then sixteen words per slot: kernel id, CTAs, entry, start, end, CTAs done, and ten
// marks that one chosen thread of the grid may set on its way (FERRIS_TL_MARK, after the wait only).
// The host fills entry and start with ones before a run.
// ---------------------------------------------------------------------------------------------
#ifdef FERRIS_TIMELINE
static __device__ unsigned long long* ferris_tl_buf;  // one per translation unit, all pointing at the same buffer
struct FerrisTl {
    unsigned long long entry;
    int slot;
};
__device__ __forceinline__ unsigned long long ferris_tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool ferris_tl_first_thread() { return threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0; }
__device__ __forceinline__ void ferris_tl_begin(FerrisTl& tl) {
    tl.slot = -1;
    if (!ferris_tl_first_thread() || !ferris_tl_buf) return;
    volatile unsigned long long* b = ferris_tl_buf;
    const int slot = (int)b[0];
    if (slot >= (int)b[1]) return;
    unsigned long long* s = ferris_tl_buf + 2 + (size_t)slot * 16;
    atomicMin(&s[2], tl.entry);
    atomicMin(&s[3], ferris_tl_now());
    tl.slot = slot;
}
__device__ __forceinline__ void ferris_tl_end(const FerrisTl& tl, int id) {
    if (!ferris_tl_first_thread() || tl.slot < 0) return;
    unsigned long long* s = ferris_tl_buf + 2 + (size_t)tl.slot * 16;
    atomicMax(&s[4], ferris_tl_now());
    const unsigned long long total = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(&s[5], 1ull) == total - 1) {
        s[0] = (unsigned long long)id;
        s[1] = total;
        __threadfence();
        atomicExch(ferris_tl_buf, (unsigned long long)(tl.slot + 1));
    }
}
__device__ __forceinline__ void ferris_tl_mark(int k) {
    if (!ferris_tl_buf) return;
    volatile unsigned long long* b = ferris_tl_buf;
    const int slot = (int)b[0];  // this launch's slot: the launches before it have completed
    if (slot < (int)b[1]) ferris_tl_buf[2 + (size_t)slot * 16 + 6 + k] = ferris_tl_now();
}
#define FERRIS_TL_MARK(cond, k) \
    do {                        \
        if (cond) ferris_tl_mark(k); \
    } while (0)
// a value of the kernel's own choice (e.g. clock cycles spent in one kind of wait) in place of a mark
__device__ __forceinline__ void ferris_tl_value(int k, unsigned long long v) {
    if (!ferris_tl_buf) return;
    volatile unsigned long long* b = ferris_tl_buf;
    const int slot = (int)b[0];
    if (slot < (int)b[1]) ferris_tl_buf[2 + (size_t)slot * 16 + 6 + k] = v;
}
#define FERRIS_TL_VALUE(cond, k, v) \
    do {                            \
        if (cond) ferris_tl_value((k), (v)); \
    } while (0)
#define FERRIS_TL_CLOCK() clock64()
#define FERRIS_TL_ENTRY() FerrisTl ferris_tl_ = {ferris_tl_now(), -1}
#define FERRIS_TL_BEGIN() ferris_tl_begin(ferris_tl_)
#define FERRIS_TL_END(id) ferris_tl_end(ferris_tl_, (id))
#define FERRIS_TIMELINE_TU(name)                                                                  \
    FERRIS_API int ferris_timeline_install_##name(unsigned long long* buf) {                      \
        return (int)cudaMemcpyToSymbol(ferris_tl_buf, &buf, sizeof(buf));                         \
    }
#else
#define FERRIS_TL_ENTRY()
#define FERRIS_TL_BEGIN()
#define FERRIS_TL_END(id)
#define FERRIS_TL_MARK(cond, k)
#define FERRIS_TL_VALUE(cond, k, v)
#define FERRIS_TL_CLOCK() 0ll
#define FERRIS_TIMELINE_TU(name)
#endif

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
