// Shared declarations of the bi8 library's translation units (not part of the public ABI).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/bi8.h"

namespace bi8 {

// Records the message returned by bi8_last_error_string() and returns `code`.
int fail(int code, const char* fmt, ...);

// Address of the per-device status word (two ints: code, detail), resolved once per device.
int* device_status_ptr();

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

#define BI8_CUDA_TRY(expr)                                                                    \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess) return ::bi8::fail(BI8_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

// The opt-in to more than 48 KiB of dynamic shared memory is an attribute of a kernel ON A DEVICE.  A launcher keeps
// one SmemOptIn per kernel instance (a function-local static) and calls ensure() before every launch: the attribute
// is set the first time the instance is used on each device, under a mutex (launchers run on several host threads).
struct SmemOptIn {
    std::mutex mu;
    size_t bytes[64] = {0};
    template <typename Kern>
    int ensure(Kern kern, size_t want) {
        int dev = 0;
        BI8_CUDA_TRY(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64) return fail(BI8_ERR_CUDA, "device ordinal %d out of range", dev);
        std::lock_guard<std::mutex> lock(mu);
        if (bytes[dev] >= want) return BI8_OK;
        BI8_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)want));
        bytes[dev] = want;
        return BI8_OK;
    }
};

// ---- launchers implemented in the other translation units -------------------------------------
int launch_quantize_rowwise(const void* x, int dt, int64_t ldx, int8_t* q, float* s, int64_t M, int64_t K,
                            int block, cudaStream_t st);
int launch_quantize_colwise(const void* x, int dt, int64_t ldx, int8_t* q, float* s, int64_t R, int64_t C,
                            int block, cudaStream_t st);
// tile quantizer (quantize_tile.cu): column-wise result, and with q_row != nullptr the row-wise result of the same input
bool quantize_tile_applicable(const void* x, int dt, int64_t ldx, const void* q_col, const void* q_row, int64_t R, int64_t C, int block);
int launch_quantize_tile(const void* x, int dt, int64_t ldx, int8_t* q_col, float* s_col, int8_t* q_row, float* s_row, int64_t R,
                         int64_t C, int block, cudaStream_t st);
// sum of the ranks' fp32 partial results over peer memory (peer_reduce.cu)
size_t peer_allreduce_buffer_bytes(int world, int64_t capacity);
int launch_peer_allreduce(void* const* peer_bufs, int rank, int world, int64_t capacity, const float* partial, int64_t M, int64_t N,
                          const void* bias, int bias_dtype, void* out, int out_dtype, unsigned wait_limit_us, cudaStream_t st);
// quantizers with the producing elementwise step in front (quantize_pre.cu); q has row pitch K
int launch_quantize_pre(int op, const void* x, const void* x2, int dt, int64_t ldx, const void* weight, float eps, int8_t* q, float* sx,
                        int64_t M, int64_t K, int block, cudaStream_t st);
// C[m, n] += R[m, n] in the type of C (C may be R)
int launch_residual_add(void* C, int64_t ldc, const void* R, int64_t ldr, int dt, int64_t M, int64_t N, cudaStream_t st);
// prefill-sized sum over ranks: reduce-scatter by peer loads, all-gather by peer stores (peer_reduce_large.cu)
size_t peer_allreduce_large_buffer_bytes(int64_t capacity);
size_t peer_allreduce_large_partial_offset();
size_t peer_allreduce_large_out_offset(int64_t capacity);
int launch_peer_allreduce_large(void* const* peer_bufs, int rank, int world, int64_t capacity, int64_t M, int64_t N, const void* bias,
                                int bias_dtype, int out_dtype, unsigned wait_limit_us, cudaStream_t st);
// rotary embedding of q and k and the append of k and v to the caches for one decode step (rope_cache.cu)
int launch_rope_cache_append(const void* qkv, int dt, const float* cis, const long long* pos, void* q_out, void* kcache, void* vcache,
                             int64_t B, int64_t H, int64_t D, int64_t max_len, cudaStream_t st);
int launch_dequantize_rowwise(const int8_t* q, const float* s, void* out, int dt, int64_t M, int64_t K,
                              int block, cudaStream_t st);

// Row-parallel layers: the fp32 result in C is this rank's partial result; where the kernel that finishes the GEMM can, it
// hands its values straight to the peer-memory reduction (peer_common.cuh) instead of leaving that to a second kernel.
struct PeerEpilogue {
    const void* args;         // const PeerArgs*
    const void* bias;
    int bias_dtype;
    void* out;                // [M, N] of out_dtype, contiguous
    int out_dtype;
    long long limit_cycles;
};

struct GemmArgs {
    const int8_t* A;
    int64_t lda;
    const int8_t* Bt;
    int64_t ldb;
    const float* sA;
    const float* sB;
    const void* bias;
    int bias_dtype;
    void* C;
    int64_t ldc;
    int out_dtype;
    int32_t* partials;  // non-null: write int32 block partial sums [nb, M, N] instead of C
    int64_t M, N, K;
    int block;
    int flags;
    void* workspace;          // optional scratch for split-K partial results
    size_t workspace_bytes;
    const void* X = nullptr;  // non-null: activations before quantization (A and sA unused), quantized on load
    int x_dtype = 0;
    int64_t ldx = 0;
    bool after_own_quantizer = false;   // the kernel launched just before is this library's decode quantizer
    unsigned wait_limit_us = 0;         // diagnostic: limit of the general kernel's bounded waits (0 = default, about 2 s)
    int skip_stage = -1;                // diagnostic: the general kernel's producer leaves this stage of its first item out
    const PeerEpilogue* peer = nullptr; // decode kernel only: reduce over the ranks inside its reduction kernel
    int64_t bias_ld = 0;                // decode kernel only: row pitch of `bias` in elements; non-zero makes it an [M, N] addend
};

bool gemm_tc_applicable(const GemmArgs& g, const char** why);
size_t gemm_tc_workspace_bytes(const GemmArgs& g);
int launch_gemm_tc(const GemmArgs& g, cudaStream_t st);
int launch_gemm_generic(const GemmArgs& g, cudaStream_t st);
bool gemm_skinny_applicable(const GemmArgs& g);
size_t gemm_skinny_workspace_bytes(const GemmArgs& g);
int launch_gemm_skinny(const GemmArgs& g, cudaStream_t st);
int launch_skinny_quantize(const void* x, int x_dtype, int64_t ldx, int8_t* q, float* sx, int64_t M, int64_t K, int block,
                           cudaStream_t st);
bool gemm_smallm_applicable(const GemmArgs& g);
int launch_gemm_smallm(const GemmArgs& g, cudaStream_t st);
int run_mma_peak_probe(int iters, float* ms, int* sm_count);

// ---- small device helpers ----------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// fp32 -> bf16 bits, round to nearest even (two values packed: lo in bits 0-15)
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

}  // namespace bi8
