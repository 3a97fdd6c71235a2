// Pieces shared by the tensor-core GEMM kernels (not part of the public ABI): the codes a bounded wait reports,
// the tensor-map encoder obtained from the driver, and the per-device facts the launchers need.
#pragma once

#include "bi8_common.cuh"
#include "sm100_ptx.cuh"

#include <cuda.h>

#include <mutex>

namespace bi8 {

constexpr int kBK = 128;   // K bytes per pipeline stage (one 128-byte swizzle row)

// codes stored in the status word's detail when a bounded wait gives up
enum WaitCode { W_EMPTY_AB = 1, W_FULL_AB = 2, W_ACC_EMPTY = 3, W_ACC_FULL = 4, W_SC_EMPTY = 5, W_SC_FULL = 6, W_PROBE = 7 };

// Raises the CTA's abort flag (a word in shared memory) and records the first failing wait in the device's
// status word.
__device__ __forceinline__ void report_timeout(int* status, uint32_t abort_flag, int code) {
    ptx::sts_u32(abort_flag, 1u);
    if (atomicCAS(status, 0, BI8_ERR_TIMEOUT) == 0) status[1] = code;
}

// ---- host side --------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// cuTensorMapEncodeTiled is a driver call and wants a context current on the calling thread.  A thread that has made no
// runtime call yet has none (an autograd worker thread whose first CUDA work is one of this library's functions; any fresh
// host thread), and the encode then fails with CUDA_ERROR_INVALID_CONTEXT: bind the current device's primary context first.
inline void ensure_current_context() {
    typedef CUresult (*GetCurrentFn)(CUcontext*);
    static GetCurrentFn get_current = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            get_current = reinterpret_cast<GetCurrentFn>(sym);
    });
    CUcontext ctx = nullptr;
    if (get_current && get_current(&ctx) == CUDA_SUCCESS && ctx != nullptr) return;
    (void)cudaFree(nullptr);          // initialises the runtime on this thread and makes the primary context current
}

// int8 [rows, K] row-major with row pitch ld bytes -> boxes of 128 K-bytes x box_rows rows, 128-byte swizzle
inline int make_operand_map(CUtensorMap* map, const int8_t* ptr, int64_t rows, int64_t K, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    ensure_current_context();
    cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return BI8_OK;
}

// fp32 scales [nb, cols] row-major (contiguous rows; cols a multiple of 4 and a 16-byte aligned base) -> boxes of
// box_cols columns x box_blocks rows, no swizzle; elements outside the tensor read as zero.
inline int make_scale_map(CUtensorMap* map, const float* ptr, int64_t nb, int64_t cols, int box_cols, int box_blocks) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    ensure_current_context();
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)nb};
    cuuint64_t gstride[1] = {(cuuint64_t)cols * 4};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_blocks};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled (scales) failed with CUresult %d", (int)r);
    return BI8_OK;
}

// Output [rows, cols] row-major of 2- or 4-byte elements with row pitch ld elements (16-byte aligned base and pitch) ->
// boxes of box_cols columns x box_rows rows, no swizzle; a store writes only the part of a box that lies inside the tensor.
inline int make_output_map(CUtensorMap* map, void* ptr, int esz, int64_t rows, int64_t cols, int64_t ld, int box_rows, int box_cols) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    ensure_current_context();
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * (cuuint64_t)esz};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, ptr, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
    return BI8_OK;
}

// ---- tensor-map cache ---------------------------------------------------------------------------------
// Encoding a tensor map is a driver call of a few microseconds; a layer calls the GEMM with the same weight and scale
// tensors every step.  A map depends only on (device, base address, extents, pitch, box), so encoded maps are kept in
// a small table guarded by a mutex and looked up by those values (a stale entry for a freed and re-used address is
// still a correct description of that address).
struct MapKey {
    int dev, kind;            // kind 0: int8 operand, 1: fp32 scales, 2 / 4: output of 2- / 4-byte elements, 5 / 6: input and int8 tiles of the tile quantizer
    const void* ptr;
    int64_t rows, cols, ld;
    int box_rows, box_cols;
    bool operator==(const MapKey& o) const {
        return dev == o.dev && kind == o.kind && ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld &&
               box_rows == o.box_rows && box_cols == o.box_cols;
    }
};

struct MapCache {
    static constexpr int kSlots = 256, kWays = 4;
    struct Entry {
        MapKey key;
        CUtensorMap map;
        bool used;
    };
    Entry table[kSlots];
    unsigned hand[kSlots / kWays];
    std::mutex mu;

    static int set_of(const MapKey& key) {
        uint64_t h = reinterpret_cast<uintptr_t>(key.ptr) * 0x9E3779B97F4A7C15ull;
        h ^= (uint64_t)key.rows * 0xC2B2AE3D27D4EB4Full + (uint64_t)key.cols * 0x165667B19E3779F9ull + (uint64_t)key.ld * 31u +
             (uint64_t)(key.box_rows * 131 + key.box_cols * 7 + key.kind * 3 + key.dev);
        return (int)((h >> 33) % (kSlots / kWays));
    }
    bool find(const MapKey& key, CUtensorMap* out) {
        const int set = set_of(key);
        std::lock_guard<std::mutex> lock(mu);
        for (int w = 0; w < kWays; ++w) {
            const Entry& e = table[set * kWays + w];
            if (e.used && e.key == key) {
                *out = e.map;
                return true;
            }
        }
        return false;
    }
    void put(const MapKey& key, const CUtensorMap& map) {
        const int set = set_of(key);
        std::lock_guard<std::mutex> lock(mu);
        Entry& e = table[set * kWays + (int)(hand[set]++ % kWays)];
        e.key = key;
        e.map = map;
        e.used = true;
    }
};
inline MapCache& map_cache() {
    static MapCache c{};
    return c;
}

inline int cached_operand_map(CUtensorMap* map, int dev, const int8_t* ptr, int64_t rows, int64_t K, int64_t ld, int box_rows) {
    const MapKey key{dev, 0, ptr, rows, K, ld, box_rows, kBK};
    if (map_cache().find(key, map)) return BI8_OK;
    const int rc = make_operand_map(map, ptr, rows, K, ld, box_rows);
    if (rc == BI8_OK) map_cache().put(key, *map);
    return rc;
}

inline int cached_scale_map(CUtensorMap* map, int dev, const float* ptr, int64_t nb, int64_t cols, int box_cols, int box_blocks) {
    const MapKey key{dev, 1, ptr, nb, cols, cols, box_blocks, box_cols};
    if (map_cache().find(key, map)) return BI8_OK;
    const int rc = make_scale_map(map, ptr, nb, cols, box_cols, box_blocks);
    if (rc == BI8_OK) map_cache().put(key, *map);
    return rc;
}

inline int cached_output_map(CUtensorMap* map, int dev, void* ptr, int esz, int64_t rows, int64_t cols, int64_t ld, int box_rows,
                             int box_cols) {
    const MapKey key{dev, esz, ptr, rows, cols, ld, box_rows, box_cols};
    if (map_cache().find(key, map)) return BI8_OK;
    const int rc = make_output_map(map, ptr, esz, rows, cols, ld, box_rows, box_cols);
    if (rc == BI8_OK) map_cache().put(key, *map);
    return rc;
}

struct DeviceInfo {
    int sms = 0;
    bool ok = false;
};
inline DeviceInfo device_info() {
    static DeviceInfo cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DeviceInfo{};
    if (!cache[dev].ok) {
        int sms = 0, major = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return DeviceInfo{};
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return DeviceInfo{};
        cache[dev].sms = sms;
        cache[dev].ok = (major == 10);
    }
    return cache[dev];
}

}  // namespace bi8
