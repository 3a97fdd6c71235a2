// extern "C" surface of libbi8.so: argument validation, dispatch, error text.  See include/bi8.h.
#include "bi8_common.cuh"
#include "peer_common.cuh"

#include <cstdarg>
#include <cstdio>
#include <mutex>

namespace bi8 {

namespace {
thread_local char g_err[512] = "";

// Per-device status word of the kernels' bounded waits: {code, detail}.
__device__ int g_status[2];
}  // namespace

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int* device_status_ptr() {
    static int* ptrs[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        fail(BI8_ERR_CUDA, "cudaGetDevice failed");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_status);
        if (e != cudaSuccess) {
            fail(BI8_ERR_CUDA, "cudaGetSymbolAddress(status): %s", cudaGetErrorString(e));
            return nullptr;
        }
        ptrs[dev] = static_cast<int*>(p);
    }
    return ptrs[dev];
}

namespace {

bool dtype_ok(int dt) { return dt == BI8_BF16 || dt == BI8_F32 || dt == BI8_F16; }
int dtype_size(int dt) { return dt == BI8_F32 ? 4 : 2; }

int check_gemm(const GemmArgs& g, bool partials) {
    if (g.M < 0 || g.N < 0 || g.K < 0) return fail(BI8_ERR_SHAPE, "gemm: negative dimension (M=%lld N=%lld K=%lld)", (long long)g.M, (long long)g.N, (long long)g.K);
    if (g.block < 1) return fail(BI8_ERR_BLOCK, "gemm: block size %d", g.block);
    if (g.M == 0 || g.N == 0) return BI8_OK;
    if (g.K > 0 && (!g.A || !g.Bt)) return fail(BI8_ERR_NULL, "gemm: null operand");
    if (g.lda < g.K || g.ldb < g.K) return fail(BI8_ERR_SHAPE, "gemm: row pitch smaller than K");
    if (partials) {
        if (!g.partials && g.K > 0) return fail(BI8_ERR_NULL, "gemm_block_partials: null output");
    } else {
        if (!g.C) return fail(BI8_ERR_NULL, "gemm: null output");
        if (g.K > 0 && (!g.sA || !g.sB)) return fail(BI8_ERR_NULL, "gemm: null scale tensor");
        if (!dtype_ok(g.out_dtype)) return fail(BI8_ERR_DTYPE, "gemm: unknown output dtype code %d", g.out_dtype);
        if (g.bias && !dtype_ok(g.bias_dtype)) return fail(BI8_ERR_DTYPE, "gemm: unknown bias dtype code %d", g.bias_dtype);
        if (g.ldc < g.N) return fail(BI8_ERR_SHAPE, "gemm: ldc smaller than N");
        if (!aligned(g.C, dtype_size(g.out_dtype))) return fail(BI8_ERR_ALIGN, "gemm: output not element aligned");
    }
    return BI8_OK;
}

int dispatch_gemm(const GemmArgs& g, cudaStream_t st) {
    const char* why = "";
    const bool tc_ok = g.K > 0 && gemm_tc_applicable(g, &why);
    if (g.flags & BI8_GEMM_FORCE_SMALLM) {
        if (!gemm_smallm_applicable(g)) return fail(BI8_ERR_ALIGN, "small-M GEMM not applicable (needs M <= 16, block 32/64/128, K %% 16 == 0, 32-byte aligned weight rows)");
        return launch_gemm_smallm(g, st);
    }
    if (g.flags & BI8_GEMM_FORCE_SKINNY) {
        if (!gemm_skinny_applicable(g))
            return fail(BI8_ERR_ALIGN, "skinny tensor-core GEMM not applicable (needs M <= 64, block 32/64/128, N %% 4 == 0, 16-byte aligned "
                                       "operand rows and weight scales, and the workspace bi8_gemm_workspace_bytes() asks for)");
        return launch_gemm_skinny(g, st);
    }
    const bool free_choice = !(g.flags & (BI8_GEMM_FORCE_TC | BI8_GEMM_FORCE_GENERIC)) && g.K > 0;
    // M <= 64: one pass over the weights on the tensor cores with exchanged operand roles (needs the workspace)
    if (free_choice && gemm_skinny_applicable(g)) return launch_gemm_skinny(g, st);
    // otherwise M <= 8 streams the weights on the CUDA cores; 9..16 would stream them twice and is faster on the
    // general tensor-core kernel
    if (free_choice && g.M <= 8 && gemm_smallm_applicable(g)) return launch_gemm_smallm(g, st);
    if (g.flags & BI8_GEMM_FORCE_TC) {
        if (!tc_ok) return fail(BI8_ERR_ALIGN, "tensor-core GEMM not applicable: %s", why);
        return launch_gemm_tc(g, st);
    }
    if ((g.flags & BI8_GEMM_FORCE_GENERIC) || !tc_ok || g.K == 0) return launch_gemm_generic(g, st);
    return launch_gemm_tc(g, st);
}

}  // namespace
}  // namespace bi8

using namespace bi8;

extern "C" {

int bi8_version(void) { return BI8_VERSION; }

const char* bi8_last_error_string(void) { return g_err; }

int bi8_device_status(int* detail) {
    int* p = device_status_ptr();
    if (!p) return BI8_ERR_CUDA;
    int host[2] = {0, 0};
    BI8_CUDA_TRY(cudaDeviceSynchronize());
    BI8_CUDA_TRY(cudaMemcpy(host, p, sizeof(host), cudaMemcpyDeviceToHost));
    if (host[0] != 0) {
        int zero[2] = {0, 0};
        BI8_CUDA_TRY(cudaMemcpy(p, zero, sizeof(zero), cudaMemcpyHostToDevice));
        if (detail) *detail = host[1];
        return fail(host[0], "a device-side bounded wait gave up (wait code %d)", host[1]);
    }
    if (detail) *detail = 0;
    return BI8_OK;
}

int bi8_quantize_rowwise(const void* x, int x_dtype, int64_t ldx, int8_t* q, float* s, int64_t M, int64_t K, int block,
                         void* stream) {
    if (!dtype_ok(x_dtype)) return fail(BI8_ERR_DTYPE, "quantize_rowwise: unknown dtype code %d", x_dtype);
    if (block < 1) return fail(BI8_ERR_BLOCK, "quantize_rowwise: block size %d", block);
    if (M < 0 || K < 0 || ldx < K) return fail(BI8_ERR_SHAPE, "quantize_rowwise: bad shape M=%lld K=%lld ldx=%lld", (long long)M, (long long)K, (long long)ldx);
    if (M == 0 || K == 0) return BI8_OK;
    if (!x || !q || !s) return fail(BI8_ERR_NULL, "quantize_rowwise: null pointer");
    if (!aligned(x, dtype_size(x_dtype)) || !aligned(s, 4)) return fail(BI8_ERR_ALIGN, "quantize_rowwise: pointer not element aligned");
    return launch_quantize_rowwise(x, x_dtype, ldx, q, s, M, K, block, static_cast<cudaStream_t>(stream));
}

int bi8_quantize_colwise(const void* x, int x_dtype, int64_t ldx, int8_t* q, float* s, int64_t R, int64_t C, int block,
                         void* stream) {
    if (!dtype_ok(x_dtype)) return fail(BI8_ERR_DTYPE, "quantize_colwise: unknown dtype code %d", x_dtype);
    if (block < 1) return fail(BI8_ERR_BLOCK, "quantize_colwise: block size %d", block);
    if (R < 0 || C < 0 || ldx < C) return fail(BI8_ERR_SHAPE, "quantize_colwise: bad shape R=%lld C=%lld ldx=%lld", (long long)R, (long long)C, (long long)ldx);
    if (R == 0 || C == 0) return BI8_OK;
    if (!x || !q || !s) return fail(BI8_ERR_NULL, "quantize_colwise: null pointer");
    if (!aligned(x, dtype_size(x_dtype)) || !aligned(s, 4)) return fail(BI8_ERR_ALIGN, "quantize_colwise: pointer not element aligned");
    return launch_quantize_colwise(x, x_dtype, ldx, q, s, R, C, block, static_cast<cudaStream_t>(stream));
}

int bi8_quantize_dual(const void* x, int x_dtype, int64_t ldx, int8_t* q_row, float* s_row, int8_t* q_col, float* s_col, int64_t R,
                      int64_t C, int block, void* stream) {
    if (!dtype_ok(x_dtype)) return fail(BI8_ERR_DTYPE, "quantize_dual: unknown dtype code %d", x_dtype);
    if (block < 1) return fail(BI8_ERR_BLOCK, "quantize_dual: block size %d", block);
    if (R < 0 || C < 0 || ldx < C) return fail(BI8_ERR_SHAPE, "quantize_dual: bad shape R=%lld C=%lld ldx=%lld", (long long)R, (long long)C, (long long)ldx);
    if (R == 0 || C == 0) return BI8_OK;
    if (!x || !q_row || !s_row || !q_col || !s_col) return fail(BI8_ERR_NULL, "quantize_dual: null pointer");
    if (!aligned(x, dtype_size(x_dtype)) || !aligned(s_row, 4) || !aligned(s_col, 4)) return fail(BI8_ERR_ALIGN, "quantize_dual: pointer not element aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (quantize_tile_applicable(x, x_dtype, ldx, q_col, q_row, R, C, block))
        return launch_quantize_tile(x, x_dtype, ldx, q_col, s_col, q_row, s_row, R, C, block, st);
    // shapes the one-pass kernel does not take: the two single-purpose quantizers, same results
    const int rc = launch_quantize_rowwise(x, x_dtype, ldx, q_row, s_row, R, C, block, st);
    if (rc != BI8_OK) return rc;
    return launch_quantize_colwise(x, x_dtype, ldx, q_col, s_col, R, C, block, st);
}

size_t bi8_peer_allreduce_buffer_bytes(int world, int64_t capacity) {
    if (world < 1 || world > 8 || capacity <= 0 || capacity % 1024 != 0) return 0;
    return peer_allreduce_buffer_bytes(world, capacity);
}

int bi8_peer_allreduce(void* const* peer_bufs, int rank, int world, int64_t capacity, const float* partial, int64_t M, int64_t N,
                       const void* bias, int bias_dtype, void* out, int out_dtype, unsigned wait_limit_us, void* stream) {
    if (!peer_bufs || !partial || !out) return fail(BI8_ERR_NULL, "peer all-reduce: null pointer");
    if (!dtype_ok(out_dtype) || (bias && !dtype_ok(bias_dtype & ~BI8_ADDEND_FULL))) return fail(BI8_ERR_DTYPE, "peer all-reduce: unknown dtype code");
    return launch_peer_allreduce(peer_bufs, rank, world, capacity, partial, M, N, bias, bias_dtype, out, out_dtype, wait_limit_us,
                                 static_cast<cudaStream_t>(stream));
}

int bi8_dequantize_rowwise(const int8_t* q, const float* s, void* out, int out_dtype, int64_t M, int64_t K, int block,
                           void* stream) {
    if (!dtype_ok(out_dtype)) return fail(BI8_ERR_DTYPE, "dequantize: unknown dtype code %d", out_dtype);
    if (block < 1) return fail(BI8_ERR_BLOCK, "dequantize: block size %d", block);
    if (M < 0 || K < 0) return fail(BI8_ERR_SHAPE, "dequantize: bad shape M=%lld K=%lld", (long long)M, (long long)K);
    if (M == 0 || K == 0) return BI8_OK;
    if (!q || !s || !out) return fail(BI8_ERR_NULL, "dequantize: null pointer");
    if (!aligned(out, dtype_size(out_dtype)) || !aligned(s, 4)) return fail(BI8_ERR_ALIGN, "dequantize: pointer not element aligned");
    return launch_dequantize_rowwise(q, s, out, out_dtype, M, K, block, static_cast<cudaStream_t>(stream));
}

size_t bi8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int block) {
    if (M <= 0 || N <= 0 || K <= 0 || (block != 32 && block != 64 && block != 128)) return 0;
    GemmArgs g{};
    g.M = M;
    g.N = N;
    g.K = K;
    g.block = block;
    const size_t a = gemm_tc_workspace_bytes(g), b = gemm_skinny_workspace_bytes(g);
    return a > b ? a : b;
}

int bi8_gemm_dequant(const int8_t* A, int64_t lda, const int8_t* Bt, int64_t ldb, const float* sA, const float* sB,
                     const void* bias, int bias_dtype, void* C, int64_t ldc, int out_dtype, int64_t M, int64_t N, int64_t K,
                     int block, void* workspace, size_t workspace_bytes, int flags, void* stream) {
    GemmArgs g{A, lda, Bt, ldb, sA, sB, bias, bias_dtype, C, ldc, out_dtype, nullptr, M, N, K, block, flags, workspace, workspace_bytes};
    int rc = check_gemm(g, false);
    if (rc != BI8_OK || M == 0 || N == 0) return rc;
    return dispatch_gemm(g, static_cast<cudaStream_t>(stream));
}

int bi8_gemm_block_partials(const int8_t* A, int64_t lda, const int8_t* Bt, int64_t ldb, int32_t* P, int64_t M, int64_t N,
                            int64_t K, int block, int flags, void* stream) {
    GemmArgs g{A, lda, Bt, ldb, nullptr, nullptr, nullptr, 0, nullptr, N, BI8_F32, P, M, N, K, block, flags, nullptr, 0};
    int rc = check_gemm(g, true);
    if (rc != BI8_OK || M == 0 || N == 0 || K == 0) return rc;
    return dispatch_gemm(g, static_cast<cudaStream_t>(stream));
}

int bi8_gemm_dequant_fused_quant(const void* x, int x_dtype, int64_t ldx, int8_t* xq, float* sx, const int8_t* Wq, int64_t ldw,
                                 const float* sW, const void* bias, int bias_dtype, void* C, int64_t ldc, int out_dtype,
                                 int64_t M, int64_t N, int64_t K, int block, void* workspace, size_t workspace_bytes, int flags,
                                 void* stream) {
    // Decode-sized M: the skinny tensor-core GEMM.  Default: a small quantizer kernel, then the GEMM launched so that its
    // set-up and first weight copies overlap the quantizer (programmatic dependent launch).  With BI8_GEMM_QUANT_IN_KERNEL,
    // or without scratch, the GEMM kernel quantizes the activations itself as it loads its stages (one kernel, slower).
    if (!dtype_ok(x_dtype)) return fail(BI8_ERR_DTYPE, "gemm_dequant_fused_quant: unknown dtype code %d", x_dtype);
    const bool forced = (flags & (BI8_GEMM_FORCE_GENERIC | BI8_GEMM_FORCE_TC | BI8_GEMM_FORCE_SMALLM)) != 0;
    if (!forced && x && M > 0 && N > 0 && K > 0 && ldx >= K && aligned(x, dtype_size(x_dtype))) {
        GemmArgs g{xq, K, Wq, ldw, sx, sW, bias, bias_dtype, C, ldc, out_dtype, nullptr, M, N, K, block, flags, workspace, workspace_bytes};
        const bool x_vec = aligned(x, 16) && (ldx * dtype_size(x_dtype)) % 16 == 0 && K % 8 == 0;   // 8 elements per load
        const bool chained = !(flags & BI8_GEMM_QUANT_IN_KERNEL) && x_vec && xq && sx && K % 16 == 0 && aligned(xq, 16) &&
                             gemm_skinny_applicable(g);
        bool in_kernel = false;
        if (!chained) {
            g.A = nullptr;
            g.sA = nullptr;
            g.X = x;
            g.x_dtype = x_dtype;
            g.ldx = ldx;
            in_kernel = gemm_skinny_applicable(g);
        }
        if (chained || in_kernel) {
            if (!Wq || !sW || !C) return fail(BI8_ERR_NULL, "gemm_dequant_fused_quant: null pointer");
            if (ldw < K || ldc < N) return fail(BI8_ERR_SHAPE, "gemm_dequant_fused_quant: row pitch smaller than the row");
            if (!dtype_ok(out_dtype) || (bias && !dtype_ok(bias_dtype))) return fail(BI8_ERR_DTYPE, "gemm_dequant_fused_quant: unknown dtype code");
            if (!aligned(C, dtype_size(out_dtype))) return fail(BI8_ERR_ALIGN, "gemm_dequant_fused_quant: output not element aligned");
            if (in_kernel) return launch_gemm_skinny(g, static_cast<cudaStream_t>(stream));
            int rc = launch_skinny_quantize(x, x_dtype, ldx, xq, sx, M, K, block, static_cast<cudaStream_t>(stream));
            if (rc != BI8_OK) return rc;
            g.after_own_quantizer = true;
            return launch_gemm_skinny(g, static_cast<cudaStream_t>(stream));
        }
    }
    // ... two kernels otherwise, through the caller's scratch
    if (M > 0 && K > 0 && (!xq || !sx))
        return fail(BI8_ERR_WORKSPACE, "gemm_dequant_fused_quant: this shape runs as quantize + GEMM and needs the xq / sx scratch");
    int rc = bi8_quantize_rowwise(x, x_dtype, ldx, xq, sx, M, K, block, stream);
    if (rc != BI8_OK) return rc;
    return bi8_gemm_dequant(xq, K, Wq, ldw, sx, sW, bias, bias_dtype, C, ldc, out_dtype, M, N, K, block, workspace,
                            workspace_bytes, flags & ~BI8_GEMM_FORCE_SKINNY, stream);
}

int bi8_quantize_rowwise_pre(int op, const void* x, const void* x2, int x_dtype, int64_t ldx, const void* weight, float eps, int8_t* q,
                             float* scales, int64_t M, int64_t K, int block, void* stream) {
    if (!dtype_ok(x_dtype)) return fail(BI8_ERR_DTYPE, "quantize_rowwise_pre: unknown dtype code %d", x_dtype);
    if (op != BI8_PRE_NONE && op != BI8_PRE_RMSNORM && op != BI8_PRE_SILU_MUL)
        return fail(BI8_ERR_SHAPE, "quantize_rowwise_pre: unknown operation code %d", op);
    if (M < 0 || K < 0 || ldx < K) return fail(BI8_ERR_SHAPE, "quantize_rowwise_pre: bad shape M %lld K %lld ldx %lld", (long long)M, (long long)K, (long long)ldx);
    if (M == 0 || K == 0) return BI8_OK;
    if (!x || !q || !scales || (op == BI8_PRE_SILU_MUL && !x2)) return fail(BI8_ERR_NULL, "quantize_rowwise_pre: null pointer");
    const size_t esz = dtype_size(x_dtype);
    if (!aligned(x, esz) || (x2 && !aligned(x2, esz)) || (weight && !aligned(weight, esz)) || !aligned(scales, 4))
        return fail(BI8_ERR_ALIGN, "quantize_rowwise_pre: pointer not element aligned");
    return launch_quantize_pre(op, x, x2, x_dtype, ldx, weight, eps, q, scales, M, K, block, static_cast<cudaStream_t>(stream));
}

int bi8_gemm_dequant_fused_pre(int op, const void* x, const void* x2, int x_dtype, int64_t ldx, const void* norm_weight, float eps,
                               int8_t* xq, float* sx, const int8_t* Wq, int64_t ldw, const float* sW, const void* bias, int bias_dtype,
                               const void* residual, int64_t ldr, void* C, int64_t ldc, int out_dtype, int64_t M, int64_t N, int64_t K,
                               int block, void* workspace, size_t workspace_bytes, int flags, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (M > 0 && K > 0 && (!xq || !sx)) return fail(BI8_ERR_WORKSPACE, "gemm_dequant_fused_pre: the xq / sx scratch is required");
    if (residual && ldr < N) return fail(BI8_ERR_SHAPE, "gemm_dequant_fused_pre: residual row pitch smaller than the row");
    if (!dtype_ok(out_dtype)) return fail(BI8_ERR_DTYPE, "gemm_dequant_fused_pre: unknown output dtype code %d", out_dtype);
    if (residual && !aligned(residual, dtype_size(out_dtype))) return fail(BI8_ERR_ALIGN, "gemm_dequant_fused_pre: residual not element aligned");
    if (M == 0 || N == 0) return BI8_OK;
    // C over the residual: only the decode path reads an element of the residual in the thread that then writes C
    const size_t osz = dtype_size(out_dtype);
    const char *c0 = static_cast<const char*>(C), *c1 = c0 + ((M - 1) * ldc + N) * osz;
    const char *r0 = static_cast<const char*>(residual), *r1 = residual ? r0 + ((M - 1) * ldr + N) * osz : r0;
    const bool overlap = residual && C && r0 < c1 && c0 < r1;
    if (overlap && (residual != C || ldr != ldc))
        return fail(BI8_ERR_SHAPE, "gemm_dequant_fused_pre: residual and C overlap without being the same tensor");
    if (op == BI8_PRE_NONE && !residual)
        return bi8_gemm_dequant_fused_quant(x, x_dtype, ldx, xq, sx, Wq, ldw, sW, bias, bias_dtype, C, ldc, out_dtype, M, N, K, block,
                                            workspace, workspace_bytes, flags, stream);
    // the decode path: this op's quantizer in the decode quantizer's place, the GEMM overlapped with it, the residual
    // added by the kernel that writes C (through the bias operand, which gets a row pitch)
    const bool forced = (flags & (BI8_GEMM_FORCE_GENERIC | BI8_GEMM_FORCE_TC | BI8_GEMM_FORCE_SMALLM | BI8_GEMM_QUANT_IN_KERNEL)) != 0;
    GemmArgs g{xq, K, Wq, ldw, sx, sW, bias, bias_dtype, C, ldc, out_dtype, nullptr, M, N, K, block, flags, workspace, workspace_bytes};
    if (!forced && K > 0 && K % 16 == 0 && aligned(xq, 16) && gemm_skinny_applicable(g)) {
        int rc = check_gemm(g, false);
        if (rc != BI8_OK) return rc;
        const bool in_kernel_residual = residual && !bias;
        if (overlap && !in_kernel_residual)
            return fail(BI8_ERR_ALIGN, "gemm_dequant_fused_pre: C may be the residual itself only without bias");
        if (in_kernel_residual) {
            g.bias = residual;
            g.bias_dtype = out_dtype;
            g.bias_ld = ldr;
        }
        const bool x_vec = dtype_ok(x_dtype) && x && aligned(x, 16) && (ldx * dtype_size(x_dtype)) % 16 == 0 && K % 8 == 0 && ldx >= K;
        if (op == BI8_PRE_NONE && x_vec) rc = launch_skinny_quantize(x, x_dtype, ldx, xq, sx, M, K, block, st);
        else rc = bi8_quantize_rowwise_pre(op, x, x2, x_dtype, ldx, norm_weight, eps, xq, sx, M, K, block, stream);
        if (rc != BI8_OK) return rc;
        // every quantizer of this library may be overlapped with the GEMM's set-up and first weight copies: none of them
        // writes weights, and the GEMM waits for the quantizer's completion before it reads the activations
        g.after_own_quantizer = true;
        rc = launch_gemm_skinny(g, st);
        if (rc != BI8_OK || !residual || in_kernel_residual) return rc;
        return launch_residual_add(C, ldc, residual, ldr, out_dtype, M, N, st);
    }
    if (overlap)
        return fail(BI8_ERR_ALIGN, "gemm_dequant_fused_pre: C may be the residual itself only on the decode path (M <= 64, N %% 4 == 0, "
                                   "K %% 16 == 0, workspace given, no bias)");
    int rc = bi8_quantize_rowwise_pre(op, x, x2, x_dtype, ldx, norm_weight, eps, xq, sx, M, K, block, stream);
    if (rc != BI8_OK) return rc;
    rc = bi8_gemm_dequant(xq, K, Wq, ldw, sx, sW, bias, bias_dtype, C, ldc, out_dtype, M, N, K, block, workspace, workspace_bytes,
                          flags & ~BI8_GEMM_QUANT_IN_KERNEL, stream);
    if (rc != BI8_OK || !residual) return rc;
    return launch_residual_add(C, ldc, residual, ldr, out_dtype, M, N, st);
}

size_t bi8_peer_allreduce_large_buffer_bytes(int world, int64_t capacity) {
    if (world < 1 || world > 8 || capacity <= 0 || capacity % 1024 != 0) return 0;
    return peer_allreduce_large_buffer_bytes(capacity);
}

size_t bi8_peer_allreduce_large_partial_offset(void) { return peer_allreduce_large_partial_offset(); }

size_t bi8_peer_allreduce_large_out_offset(int64_t capacity) { return peer_allreduce_large_out_offset(capacity); }

int bi8_peer_allreduce_large(void* const* peer_bufs, int rank, int world, int64_t capacity, int64_t M, int64_t N, const void* bias,
                             int bias_dtype, int out_dtype, unsigned wait_limit_us, void* stream) {
    if (!peer_bufs) return fail(BI8_ERR_NULL, "peer all-reduce: null pointer");
    if (!dtype_ok(out_dtype) || (bias && !dtype_ok(bias_dtype & ~BI8_ADDEND_FULL))) return fail(BI8_ERR_DTYPE, "peer all-reduce: unknown dtype code");
    return launch_peer_allreduce_large(peer_bufs, rank, world, capacity, M, N, bias, bias_dtype, out_dtype, wait_limit_us,
                                       static_cast<cudaStream_t>(stream));
}

int bi8_row_parallel_linear_pre(int op, const void* x, const void* x2, int x_dtype, int64_t ldx, const void* norm_weight, float eps,
                                int8_t* xq, float* sx, const int8_t* Wq, int64_t ldw, const float* sW, float* partial, int64_t M, int64_t N,
                                int64_t K, int block, void* workspace, size_t workspace_bytes, void* const* peer_bufs, int rank, int world,
                                int64_t capacity, const void* bias, int bias_dtype, void* out, int out_dtype, unsigned wait_limit_us,
                                int flags, void* stream) {
    if (!x || !xq || !sx || !Wq || !sW || !partial || !peer_bufs || !out) return fail(BI8_ERR_NULL, "row_parallel_linear: null pointer");
    if (!dtype_ok(x_dtype) || !dtype_ok(out_dtype) || (bias && !dtype_ok(bias_dtype & ~BI8_ADDEND_FULL)))
        return fail(BI8_ERR_DTYPE, "row_parallel_linear: unknown dtype code");
    if (M <= 0 || N <= 0 || K <= 0 || ldx < K || ldw < K) return fail(BI8_ERR_SHAPE, "row_parallel_linear: bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    if (!aligned(partial, 16) || !aligned(out, 16)) return fail(BI8_ERR_ALIGN, "row_parallel_linear: partial and out must be 16-byte aligned");
    PeerArgs pa;
    int rc = make_peer_args(&pa, peer_bufs, rank, world, capacity, M, N);
    if (rc != BI8_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool forced = (flags & (BI8_GEMM_FORCE_GENERIC | BI8_GEMM_FORCE_TC | BI8_GEMM_FORCE_SMALLM | BI8_GEMM_QUANT_IN_KERNEL)) != 0;
    const bool x_vec = aligned(x, 16) && (ldx * dtype_size(x_dtype)) % 16 == 0;
    if (!forced && (x_vec || op != BI8_PRE_NONE) && K % 16 == 0 && aligned(xq, 16)) {
        // decode-sized M: quantizer, weight-streaming GEMM, and a reduction kernel that sums the tile parts AND the ranks
        GemmArgs g{xq, K, Wq, ldw, sx, sW, nullptr, 0, partial, N, BI8_F32, nullptr, M, N, K, block, flags, workspace, workspace_bytes};
        if (gemm_skinny_applicable(g)) {
            PeerEpilogue pe{&pa, bias, bias_dtype, out, out_dtype, peer_wait_limit_cycles(wait_limit_us)};
            if (op == BI8_PRE_NONE) rc = launch_skinny_quantize(x, x_dtype, ldx, xq, sx, M, K, block, st);
            else rc = bi8_quantize_rowwise_pre(op, x, x2, x_dtype, ldx, norm_weight, eps, xq, sx, M, K, block, stream);
            if (rc != BI8_OK) return rc;
            g.after_own_quantizer = true;
            g.peer = &pe;
            return launch_gemm_skinny(g, st);
        }
    }
    // other shapes: the layer's two steps into `partial`, then the stand-alone reduction
    rc = bi8_gemm_dequant_fused_pre(op, x, x2, x_dtype, ldx, norm_weight, eps, xq, sx, Wq, ldw, sW, nullptr, 0, nullptr, 0, partial, N,
                                    BI8_F32, M, N, K, block, workspace, workspace_bytes, flags, stream);
    if (rc != BI8_OK) return rc;
    return launch_peer_allreduce(peer_bufs, rank, world, capacity, partial, M, N, bias, bias_dtype, out, out_dtype, wait_limit_us, st);
}

int bi8_row_parallel_linear(const void* x, int x_dtype, int64_t ldx, int8_t* xq, float* sx, const int8_t* Wq, int64_t ldw,
                            const float* sW, float* partial, int64_t M, int64_t N, int64_t K, int block, void* workspace,
                            size_t workspace_bytes, void* const* peer_bufs, int rank, int world, int64_t capacity, const void* bias,
                            int bias_dtype, void* out, int out_dtype, unsigned wait_limit_us, int flags, void* stream) {
    return bi8_row_parallel_linear_pre(BI8_PRE_NONE, x, nullptr, x_dtype, ldx, nullptr, 0.0f, xq, sx, Wq, ldw, sW, partial, M, N, K, block,
                                       workspace, workspace_bytes, peer_bufs, rank, world, capacity, bias, bias_dtype, out, out_dtype,
                                       wait_limit_us, flags, stream);
}

int bi8_rope_cache_append(const void* qkv, int dtype, const float* cis, const long long* pos, void* q_out, void* kcache, void* vcache,
                          int64_t B, int64_t H, int64_t D, int64_t max_len, void* stream) {
    if (dtype != BI8_BF16 && dtype != BI8_F16) return fail(BI8_ERR_DTYPE, "rope_cache_append: bf16 or fp16 activations (got code %d)", dtype);
    if (B < 0 || H < 0 || D < 0 || D % 2 != 0 || max_len <= 0 || B > 0x7fffffff || H > 0x7fffffff || D > 0x7fffffff || max_len > 0x7fffffff)
        return fail(BI8_ERR_SHAPE, "rope_cache_append: bad shape B %lld H %lld D %lld max_len %lld", (long long)B, (long long)H, (long long)D, (long long)max_len);
    if (B == 0 || H == 0 || D == 0) return BI8_OK;
    if (!qkv || !cis || !pos || !q_out || !kcache || !vcache) return fail(BI8_ERR_NULL, "rope_cache_append: null pointer");
    if (!aligned(qkv, 4) || !aligned(q_out, 4) || !aligned(kcache, 4) || !aligned(vcache, 4) || !aligned(cis, 8) || !aligned(pos, 8))
        return fail(BI8_ERR_ALIGN, "rope_cache_append: pointer not aligned to an element pair");
    return launch_rope_cache_append(qkv, dtype, cis, pos, q_out, kcache, vcache, B, H, D, max_len, static_cast<cudaStream_t>(stream));
}

int bi8_stream_capture_id(void* stream, unsigned long long* id) {
    if (!id) return fail(BI8_ERR_NULL, "stream_capture_id: null output");
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    unsigned long long cid = 0;
    BI8_CUDA_TRY(cudaStreamGetCaptureInfo(static_cast<cudaStream_t>(stream), &st, &cid));
    *id = (st == cudaStreamCaptureStatusActive) ? cid : 0ull;
    return BI8_OK;
}

int bi8_gemm_wait_selftest(const int8_t* A, int64_t lda, const int8_t* Bt, int64_t ldb, const float* sA, const float* sB, void* C,
                           int64_t ldc, int out_dtype, int64_t M, int64_t N, int64_t K, int block, unsigned wait_limit_us,
                           int skip_stage, void* stream) {
    GemmArgs g{A, lda, Bt, ldb, sA, sB, nullptr, 0, C, ldc, out_dtype, nullptr, M, N, K, block, BI8_GEMM_FORCE_TC, nullptr, 0};
    int rc = check_gemm(g, false);
    if (rc != BI8_OK) return rc;
    if (M == 0 || N == 0 || K == 0) return fail(BI8_ERR_SHAPE, "gemm_wait_selftest: empty problem");
    if (wait_limit_us > 2000000u) return fail(BI8_ERR_LIMIT, "gemm_wait_selftest: wait limit above two seconds");
    g.wait_limit_us = wait_limit_us;
    g.skip_stage = skip_stage;
    return dispatch_gemm(g, static_cast<cudaStream_t>(stream));
}

int bi8_mma_peak_probe(int iters, float* ms, int* sm_count) {
    if (!ms) return fail(BI8_ERR_NULL, "mma_peak_probe: null output");
    return run_mma_peak_probe(iters, ms, sm_count);
}

}  // extern "C"
