// Error text of the C ABI and a few queries about the device.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "sm100.cuh"

static thread_local char g_error[512] = "";

void ferris_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

FERRIS_API const char* ferris_last_error() { return g_error; }

// Programmatic dependent launch is on unless the environment says FERRIS_PDL=0.
static int g_pdl = -1;
bool ferris_pdl_enabled() {
    if (g_pdl < 0) {
        const char* v = getenv("FERRIS_PDL");
        g_pdl = (v && v[0] == '0') ? 0 : 1;
    }
    return g_pdl != 0;
}
FERRIS_API void ferris_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// Compute capability of the current device as major * 10 + minor, or a negative cudaError_t.
FERRIS_API int ferris_device_arch() {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) {
        ferris_set_error("%s", cudaGetErrorString(e));
        return -(int)e;
    }
    return major * 10 + minor;
}

FERRIS_API int ferris_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return n;
}

// ---------------------------------------------------------------------------------------------
// The status word that kernels with bounded waits write when a wait runs out.
// ---------------------------------------------------------------------------------------------
static __device__ int g_status_word = 0;
static int* g_status_ptr = nullptr;

int* ferris_status_ptr() {
    if (!g_status_ptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) == cudaSuccess) g_status_ptr = (int*)p;
    }
    return g_status_ptr;
}

// Reads and clears the status word (synchronises the device).  0 = no kernel reported a fault.
FERRIS_API int ferris_kernel_status() {
    int* p = ferris_status_ptr();
    if (!p) return -1;
    int v = 0, zero = 0;
    if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
    return v;
}

// ---------------------------------------------------------------------------------------------
// Tensor maps.  cuTensorMapEncodeTiled is reached through the runtime's driver entry point, so the
// library links against no driver stub.
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

int ferris_encode_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                                uint32_t box_rows, uint32_t box_cols);
int ferris_encode_tensor_map_2d_f32(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                                    uint64_t row_stride, uint32_t box_rows);

// The launchers make a tensor map for their activations at every call, and the same few buffers of the workspace
// come back step after step: a small direct-mapped table of the maps made last saves the driver call.
namespace {
struct MapKey {
    const void* base;
    uint64_t rows, cols, row_stride;
    uint32_t box_rows, box_cols, kind;
};
struct MapSlot {
    MapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int MAP_SLOTS = 256;
MapSlot g_map_slots[MAP_SLOTS];
inline bool same(const MapKey& a, const MapKey& b) {
    return a.base == b.base && a.rows == b.rows && a.cols == b.cols && a.row_stride == b.row_stride &&
           a.box_rows == b.box_rows && a.box_cols == b.box_cols && a.kind == b.kind;
}
inline MapSlot& slot_of(const MapKey& k) {
    uint64_t h = (uint64_t)(uintptr_t)k.base * 0x9E3779B97F4A7C15ull ^ (k.rows * 31 + k.cols * 131 + k.box_rows * 7 + k.kind);
    return g_map_slots[(h >> 32) % MAP_SLOTS];
}
}  // namespace

int ferris_make_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                              uint32_t box_rows, uint32_t box_cols) {
    const MapKey key = {base, rows, cols, row_stride, box_rows, box_cols, 0u};
    MapSlot& slot = slot_of(key);
    if (slot.used && same(slot.key, key)) {
        *map = slot.map;
        return FERRIS_OK;
    }
    int rc = ferris_encode_tensor_map_2d(map, base, rows, cols, row_stride, box_rows, box_cols);
    if (rc == FERRIS_OK) slot = {key, *map, true};
    return rc;
}

int ferris_encode_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                                uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) FERRIS_REFUSE("tensor map: the driver offers no cuTensorMapEncodeTiled");
    if (((uintptr_t)base & 15) || ((row_stride * 2) & 15) || box_cols * 2 != 128 || box_rows == 0 || box_rows > 256)
        FERRIS_REFUSE("tensor map: base %p, row stride %llu, box %u x %u do not meet the alignment rules", base,
                      (unsigned long long)row_stride, box_rows, box_cols);
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) FERRIS_REFUSE("tensor map: cuTensorMapEncodeTiled failed with %d", (int)r);
    return FERRIS_OK;
}

// A bf16 matrix [rows, cols] (cols a multiple of 64) seen as [rows][64-column blocks][64]: one box is `box_rows` rows of
// `box_kblocks` consecutive blocks, and lands in shared memory as box_rows x box_kblocks lines of 128 bytes (line
// row * box_kblocks + block), swizzled by the line's number.  One copy thus brings what box_kblocks copies of the
// 2-D map bring; with an odd box_kblocks the eight rows of one block fall into eight different swizzle phases.
int ferris_make_tensor_map_kblocks(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                                   uint32_t box_rows, uint32_t box_kblocks) {
    const MapKey key = {base, rows, cols, row_stride, box_rows, box_kblocks, 2u};
    MapSlot& slot = slot_of(key);
    if (slot.used && same(slot.key, key)) {
        *map = slot.map;
        return FERRIS_OK;
    }
    EncodeTiledFn fn = encode_tiled();
    if (!fn) FERRIS_REFUSE("tensor map: the driver offers no cuTensorMapEncodeTiled");
    if (((uintptr_t)base & 15) || ((row_stride * 2) & 15) || (cols & 63) || box_rows == 0 || box_rows > 256 ||
        box_kblocks == 0 || box_kblocks > 256)
        FERRIS_REFUSE("tensor map: base %p, row stride %llu, %llu columns, box %u rows x %u blocks do not meet the rules", base,
                      (unsigned long long)row_stride, (unsigned long long)cols, box_rows, box_kblocks);
    cuuint64_t dims[3] = {64, cols / 64, rows};
    cuuint64_t strides[2] = {128, row_stride * 2};
    cuuint32_t box[3] = {64, box_kblocks, box_rows};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) FERRIS_REFUSE("tensor map: cuTensorMapEncodeTiled (3-D) failed with %d", (int)r);
    slot = {key, *map, true};
    return FERRIS_OK;
}

// Two bf16 matrices [rows, cols] that lie `plane_bytes` apart, as one 3-D tensor (cols, rows, 2): a box is 64 columns x
// `box_rows` rows of both, and lands in shared memory as the first matrix's box followed by the second's, each
// swizzled like a 2-D box.
int ferris_make_tensor_map_planes(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t plane_bytes,
                                  uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) FERRIS_REFUSE("tensor map: the driver offers no cuTensorMapEncodeTiled");
    if (((uintptr_t)base & 15) || ((cols * 2) & 15) || (plane_bytes & 15) || plane_bytes < rows * cols * 2 || box_rows == 0 ||
        box_rows > 256 || (box_rows & 7))
        FERRIS_REFUSE("tensor map: base %p, %llu columns, planes %llu bytes apart, box of %u rows do not meet the rules", base,
                      (unsigned long long)cols, (unsigned long long)plane_bytes, box_rows);
    cuuint64_t dims[3] = {cols, rows, 2};
    cuuint64_t strides[2] = {cols * 2, plane_bytes};
    cuuint32_t box[3] = {64, box_rows, 2};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) FERRIS_REFUSE("tensor map: cuTensorMapEncodeTiled (planes) failed with %d", (int)r);
    return FERRIS_OK;
}

int ferris_make_tensor_map_2d_f32(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                                  uint64_t row_stride, uint32_t box_rows) {
    const MapKey key = {base, rows, cols, row_stride, box_rows, 32u, 1u};
    MapSlot& slot = slot_of(key);
    if (slot.used && same(slot.key, key)) {
        *map = slot.map;
        return FERRIS_OK;
    }
    int rc = ferris_encode_tensor_map_2d_f32(map, base, rows, cols, row_stride, box_rows);
    if (rc == FERRIS_OK) slot = {key, *map, true};
    return rc;
}

int ferris_encode_tensor_map_2d_f32(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                                    uint64_t row_stride, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) FERRIS_REFUSE("tensor map: the driver offers no cuTensorMapEncodeTiled");
    if (((uintptr_t)base & 15) || ((row_stride * 4) & 15) || box_rows == 0 || box_rows > 256)
        FERRIS_REFUSE("tensor map: base %p, row stride %llu, box rows %u do not meet the alignment rules", base,
                      (unsigned long long)row_stride, box_rows);
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride * 4};
    cuuint32_t box[2] = {32, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) FERRIS_REFUSE("tensor map: cuTensorMapEncodeTiled failed with %d", (int)r);
    return FERRIS_OK;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is a driver call; the launchers would make it at every launch.
// This remembers, per kernel and device, the largest size already allowed.
namespace {
struct SmemAllowance {
    const void* fn;
    int device;
    size_t bytes;
};
constexpr int ALLOWANCES = 256;
SmemAllowance g_allowances[ALLOWANCES];
int g_allowance_count = 0;
}  // namespace

int ferris_allow_dynamic_smem(const void* fn, size_t bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        ferris_set_error("%s", cudaGetErrorString(e));
        return (int)e;
    }
    SmemAllowance* hit = nullptr;
    for (int i = 0; i < g_allowance_count; ++i)
        if (g_allowances[i].fn == fn && g_allowances[i].device == dev) {
            hit = &g_allowances[i];
            break;
        }
    if (hit && hit->bytes >= bytes) return FERRIS_OK;
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) {
        ferris_set_error("%s", cudaGetErrorString(e));
        return (int)e;
    }
    if (hit)
        hit->bytes = bytes;
    else if (g_allowance_count < ALLOWANCES)
        g_allowances[g_allowance_count++] = {fn, dev, bytes};
    return FERRIS_OK;
}
