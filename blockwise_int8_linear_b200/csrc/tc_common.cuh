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

// int8 [rows, K] row-major with row pitch ld bytes -> boxes of 128 K-bytes x box_rows rows, 128-byte swizzle
inline int make_operand_map(CUtensorMap* map, const int8_t* ptr, int64_t rows, int64_t K, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
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
