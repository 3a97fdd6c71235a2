// bi8_gemm_dequant_static: the block GEMM for callers that cannot hand over a workspace.
//
// Who needs it: code that has no way to obtain device memory at the moment of the call.  Typical cases are a
// serving loop that took its whole memory budget at start-up and must not call cudaMalloc afterwards (the call
// synchronises the device and can fail once the pool is spent), a plugin inside a host runtime that owns the
// allocator and gives third-party code no access to it, and embedded callers that are only allowed a fixed
// memory footprint.  For small M the GEMM divides K over several work items (split-K) and needs scratch for the
// fp32 partial results; bi8_gemm_dequant expects the caller to supply it.  This entry point supplies it itself
// from a fixed array that lives inside the library.
//
// The array is a file-scope __device__ array of kScratchBytes: every GPU that loads the library holds that much
// memory until the process exits.  A problem whose split-K plan needs more is rejected with BI8_ERR_LIMIT.
// Nothing here (or below it) calls cudaMalloc, cudaFree or an allocating library routine.
//
// In host code the array's name is only a handle; the kernels need its device address, which
// cudaGetSymbolAddress returns for the device that is current.  The first call on each device does that
// look-up; make that first call outside any stream capture.  All calls share the one array: the GEMM overwrites
// every partial result it later reads, so nothing has to be cleared between calls, but two calls that may run
// concurrently on the same GPU (different streams, different threads) race on it and must be serialised by the
// caller.
#include "bi8_common.cuh"

#include <mutex>

namespace bi8 {
namespace {

constexpr size_t kScratchBytes = (size_t)8 << 20;   // 8 MiB: covers the split-K plans of decode-sized batches (M <= 64 on the 7B projection shapes)
__device__ __align__(256) unsigned char g_gemm_scratch[kScratchBytes];

// Device address of the scratch array on the current device (resolved once per device).
void* scratch_ptr() {
    static void* ptrs[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        fail(BI8_ERR_CUDA, "gemm_dequant_static: cudaGetDevice failed");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_gemm_scratch);
        if (e != cudaSuccess) {
            fail(BI8_ERR_CUDA, "gemm_dequant_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        ptrs[dev] = p;
    }
    return ptrs[dev];
}

}  // namespace
}  // namespace bi8

extern "C" {

size_t bi8_gemm_static_scratch_bytes(void) { return bi8::kScratchBytes; }

int bi8_gemm_dequant_static(const int8_t* A, int64_t lda, const int8_t* Bt, int64_t ldb, const float* sA, const float* sB,
                            const void* bias, int bias_dtype, void* C, int64_t ldc, int out_dtype, int64_t M, int64_t N,
                            int64_t K, int block, int flags, void* stream) {
    // the plan that cannot be left out: split-K of the general kernel.  (The decode kernel for M <= 64 asks for more
    // rows of scratch as M grows; where the array does not hold that, the dispatcher simply takes the general kernel.)
    bi8::GemmArgs shape{};
    shape.M = M;
    shape.N = N;
    shape.K = K;
    shape.block = block;
    const size_t need = (M > 0 && N > 0 && K > 0 && (block == 32 || block == 64 || block == 128)) ? bi8::gemm_tc_workspace_bytes(shape) : 0;
    if (need > bi8::kScratchBytes)
        return bi8::fail(BI8_ERR_LIMIT,
                         "gemm_dequant_static: this shape needs %zu bytes of split-K scratch, the built-in array holds %zu; "
                         "use bi8_gemm_dequant with a caller workspace",
                         need, bi8::kScratchBytes);
    // The array is offered to the dispatcher at its full size.  That is safe because every kernel that takes scratch
    // checks the size it is given against its own plan before using it: gemm_skinny_applicable() compares
    // workspace_bytes with gemm_skinny_workspace_bytes() and declines when the array is too small (the general kernel
    // then runs, whose plan was checked above), and launch_gemm_tc() runs unsplit unless workspace_bytes covers its plan.
    void* scratch = nullptr;
    size_t given = 0;
    if (bi8_gemm_workspace_bytes(M, N, K, block) > 0) {
        scratch = bi8::scratch_ptr();
        if (!scratch) return BI8_ERR_CUDA;
        given = bi8::kScratchBytes;
    }
    return bi8_gemm_dequant(A, lda, Bt, ldb, sA, sB, bias, bias_dtype, C, ldc, out_dtype, M, N, K, block, scratch, given, flags,
                            stream);
}

}  // extern "C"
