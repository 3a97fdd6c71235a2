/* bi8 — blockwise-int8 linear hot path for NVIDIA B200 (sm_100a), C ABI.
 *
 * One shared library, libbi8.so, replaces the three device kernels of the reference project and
 * their Python launch wrappers.  Every entry point takes plain device pointers, sizes and a
 * cudaStream_t (passed as void*), enqueues its work on that stream and returns an int status
 * without synchronising.  Unless a function's comment says otherwise the library owns no device
 * memory: inputs, outputs and workspaces are allocated by the caller.
 *
 * Layout contract (the reference's):
 *   quantized values  int8  [rows, K]          row-major, K contiguous
 *   block scales      fp32  [ceil(K/block), rows]   ("state" tensors; transposed on purpose)
 *   a block is `block` consecutive elements of one row; the K tail counts as zeros.
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   triton_functions.py:411-423  quantize_block_rowwise            -> bi8_quantize_rowwise
 *   triton_functions.py:492-500  dequantize_block_rowwise          -> bi8_dequantize_rowwise
 *   triton_functions.py:142-168  int8_matmul_block64_rowwise_dequantize -> bi8_gemm_dequant
 *   block_linear.py:93-94,100-103  X.t().contiguous() + quantize   -> bi8_quantize_colwise
 */
#ifndef BI8_H_
#define BI8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define BI8_API __attribute__((visibility("default")))
#else
#define BI8_API
#endif

#define BI8_VERSION 100

/* status codes (0 = ok, negative = error; text via bi8_last_error_string) */
#define BI8_OK 0
#define BI8_ERR_DTYPE (-1)      /* unsupported element type code */
#define BI8_ERR_BLOCK (-2)      /* block size < 1 */
#define BI8_ERR_ALIGN (-3)      /* pointer / stride alignment the entry point cannot handle */
#define BI8_ERR_SHAPE (-4)      /* negative or inconsistent sizes */
#define BI8_ERR_CUDA (-5)       /* a CUDA runtime / driver call failed */
#define BI8_ERR_TIMEOUT (-6)    /* a device-side bounded wait gave up (read by bi8_device_status) */
#define BI8_ERR_WORKSPACE (-7)  /* workspace missing or too small */
#define BI8_ERR_NULL (-8)       /* required pointer is null */
#define BI8_ERR_LIMIT (-9)      /* size beyond a documented fixed limit */

/* element type codes for floating-point tensors */
#define BI8_BF16 0
#define BI8_F32 1
#define BI8_F16 2

/* flags for bi8_gemm_dequant */
#define BI8_GEMM_DEFAULT 0
#define BI8_GEMM_FORCE_GENERIC 1   /* CUDA-core kernel even where the tensor-core kernel applies */
#define BI8_GEMM_FORCE_TC 2        /* fail with BI8_ERR_ALIGN instead of falling back */
#define BI8_GEMM_NO_SEED 4         /* tensor-core kernel: convert partial sums with cvt instead of seeded TMEM */
#define BI8_GEMM_FORCE_SMALLM 8    /* weight-streaming CUDA-core kernel, M <= 16 (the default choice for M <= 8) */
#define BI8_GEMM_FORCE_SKINNY 16   /* weight-streaming tensor-core kernel with exchanged operand roles, M <= 64 */
#define BI8_GEMM_QUANT_IN_KERNEL 32 /* bi8_gemm_dequant_fused_quant, M <= 32: quantize inside the GEMM kernel */

BI8_API int bi8_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
BI8_API const char* bi8_last_error_string(void);

/* Reads and clears the device-side status word of the current device (synchronises the device).
 * 0 = no kernel reported a problem; otherwise BI8_ERR_TIMEOUT (a bounded mbarrier wait gave up;
 * *detail receives the kernel-specific code of the first wait that gave up). */
BI8_API int bi8_device_status(int* detail);

/* Replaces quantize_block_rowwise (triton_functions.py:411-423, kernel 382-406).
 * x [M,K] of x_dtype, row stride ldx elements, K contiguous.  Writes q [M,K] int8 (contiguous) and
 * s [ceil(K/block), M] fp32.  scale = max|x| over the block (fp32); q = rint(127*(x/scale)) with an
 * IEEE fp32 divide, a separate fp32 multiply and round-half-even; an all-zero block gives scale 0, q 0. */
BI8_API int bi8_quantize_rowwise(const void* x, int x_dtype, int64_t ldx, int8_t* q, float* s,
                         int64_t M, int64_t K, int block, void* stream);

/* Replaces "t = x.t().contiguous(); quantize_block_rowwise(t)" (block_linear.py:93-94, 100-103) in one
 * pass.  x [R,C] of x_dtype, row stride ldx.  Writes q [C,R] int8 (the transpose, contiguous) and
 * s [ceil(R/block), C]: blocks run down the columns of x.  Bit-identical to the two-step form. */
BI8_API int bi8_quantize_colwise(const void* x, int x_dtype, int64_t ldx, int8_t* q, float* s,
                         int64_t R, int64_t C, int block, void* stream);

/* Both quantizations of one tensor from a single read: q_row [R,C] / s_row [ceil(C/block), R] as bi8_quantize_rowwise
 * gives them and q_col [C,R] / s_col [ceil(R/block), C] as bi8_quantize_colwise gives them, bit for bit.  Replaces the pairs
 * of calls at block_linear.py:78 + 100-101 (X: forward and weight gradient) and 92 + 102-103 (the output gradient). */
BI8_API int bi8_quantize_dual(const void* x, int x_dtype, int64_t ldx, int8_t* q_row, float* s_row, int8_t* q_col, float* s_col,
                      int64_t R, int64_t C, int block, void* stream);

/* Replaces dequantize_block_rowwise (triton_functions.py:492-500, kernel 467-490).
 * out[m,k] = cast((s[k/block, m] * float(q[m,k])) * fl32(1/127)), out [M,K] contiguous of out_dtype. */
BI8_API int bi8_dequantize_rowwise(const int8_t* q, const float* s, void* out, int out_dtype,
                           int64_t M, int64_t K, int block, void* stream);

/* Replaces int8_matmul_block64_rowwise_dequantize (triton_functions.py:142-168, kernel 69-139).
 *   C[m,n] = cast( sum_j  sB[j,n] * sA[j,m] * float(P_j[m,n]) / 127^2 )  (+ cast(bias[n]) in the output type)
 *   P_j = A[:, j*block:(j+1)*block] . Bt[:, j*block:(j+1)*block]^T   exactly, in int32.
 * A  [M,K] int8, row stride lda.  Bt [N,K] int8, row stride ldb — the reference's `b` operand is the
 * transposed view Bt^T with strides (1, ldb).  sA [ceil(K/block), M], sB [ceil(K/block), N] fp32.
 * bias [N] of bias_dtype or NULL.  C [M,N] of out_dtype, row stride ldc.
 * workspace: bi8_gemm_workspace_bytes(M,N,K,block) bytes of 16-byte aligned device memory (may be NULL when that
 * is 0; without it small-M shapes run on slower kernels).  It is plain scratch: nothing has to be cleared, every
 * call overwrites what it later reads; calls that may run concurrently need separate workspaces.
 * The int32 partial sums are exact.  The fp32 accumulation of the tensor-core kernel for M > 64 evaluates a term as
 * sB * fl(P * s) with s = sA/127^2 rounded to fp32 and then to 22 significant bits (relative error of s at most
 * 2^-24 + 2^-22), one rounding for P*s and one for the fused multiply-add into the sum, where the reference rounds
 * three times per term; the result stays within 12 * 2^-24 * sum_j |term_j| of the reference's.  The kernels for
 * M <= 64 and the CUDA-core kernel evaluate every term in the reference's order. */
BI8_API int bi8_gemm_dequant(const int8_t* A, int64_t lda, const int8_t* Bt, int64_t ldb,
                     const float* sA, const float* sB, const void* bias, int bias_dtype,
                     void* C, int64_t ldc, int out_dtype, int64_t M, int64_t N, int64_t K, int block,
                     void* workspace, size_t workspace_bytes, int flags, void* stream);

BI8_API size_t bi8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int block);

/* bi8_gemm_dequant for callers that cannot provide a workspace because they cannot allocate device memory when
 * they call: a serving loop that must not touch cudaMalloc after start-up, a plugin whose host runtime owns the
 * allocator, a caller with a fixed memory footprint.  (No counterpart in the reference, whose wrappers allocate
 * with torch on every call.)  The split-K scratch comes from a fixed 8 MiB array inside the library (reported by
 * bi8_gemm_static_scratch_bytes; every GPU that loads the library holds it until exit); a shape whose plan needs
 * more returns BI8_ERR_LIMIT.  No cudaMalloc/cudaFree or allocating library call is made.  The first call on a
 * device looks up the array's device address: make it outside any stream capture.  All calls share the array
 * (nothing needs clearing between calls); calls that can overlap on one GPU race on it and must be serialised by
 * the caller.  Arguments and results are those of bi8_gemm_dequant (bit-identical where both select the same kernel;
 * for 33 <= M <= 64 this entry point's scratch is too small for the decode kernel and the general kernel runs). */
BI8_API int bi8_gemm_dequant_static(const int8_t* A, int64_t lda, const int8_t* Bt, int64_t ldb,
                            const float* sA, const float* sB, const void* bias, int bias_dtype,
                            void* C, int64_t ldc, int out_dtype, int64_t M, int64_t N, int64_t K, int block,
                            int flags, void* stream);
BI8_API size_t bi8_gemm_static_scratch_bytes(void);

/* Diagnostic twin of bi8_gemm_dequant (same loads and tensor-core instructions): writes the exact
 * int32 partial sums P [ceil(K/block), M, N] instead of the scaled result (triton_functions.py:115). */
BI8_API int bi8_gemm_block_partials(const int8_t* A, int64_t lda, const int8_t* Bt, int64_t ldb, int32_t* P,
                            int64_t M, int64_t N, int64_t K, int block, int flags, void* stream);

/* Forward of the layer in one call (block_linear.py:78-80 / 141-143): quantize-on-load GEMM.  x [M,K] of x_dtype, row
 * stride ldx, is quantized per row and block exactly as bi8_quantize_rowwise does and multiplied with the
 * pre-quantized weights Wq [N,K] / sW; the result equals bi8_quantize_rowwise followed by bi8_gemm_dequant.
 * For M <= 64 (N a multiple of 4, K a multiple of 16, 16-byte aligned rows, workspace given) the weight-streaming
 * tensor-core GEMM runs behind a small quantizer kernel and is launched so that its set-up and first weight
 * loads overlap that kernel; with BI8_GEMM_QUANT_IN_KERNEL (or without scratch; M <= 32) the GEMM kernel itself quantizes
 * the activations as it loads its stages: one kernel, no scratch, but measured slower.  Every other shape runs the
 * standalone quantizer and the GEMM back to back.  xq [M,K] int8 and sx [ceil(K/block),M] fp32 are scratch, which
 * may be NULL only when the M <= 32 conditions hold.  The scratch contents after the call are
 * unspecified.  workspace as for bi8_gemm_dequant. */
BI8_API int bi8_gemm_dequant_fused_quant(const void* x, int x_dtype, int64_t ldx, int8_t* xq, float* sx,
                                 const int8_t* Wq, int64_t ldw, const float* sW, const void* bias, int bias_dtype,
                                 void* C, int64_t ldc, int out_dtype, int64_t M, int64_t N, int64_t K, int block,
                                 void* workspace, size_t workspace_bytes, int flags, void* stream);

/* The elementwise step that produces a projection's input, fused in front of the row-wise quantizer (no counterpart in the
 * reference, whose layers quantize a tensor another kernel wrote just before: block_linear.py:141).  The value of every
 * element is rounded to x_dtype exactly where the separate kernel would have stored it, then quantized with
 * bi8_quantize_rowwise's arithmetic, so q / scales equal bi8_quantize_rowwise of that rounded tensor.
 *   BI8_PRE_NONE      y = x                                                      (the plain quantizer)
 *   BI8_PRE_RMSNORM   y = cast(x * rsqrt(sum_k(x^2) / K + eps) [* weight[k]])    fp32 arithmetic, one rounding; weight may
 *                     be NULL, else [K] of x_dtype.  The sum of squares is taken in a fixed order (same bits on every call).
 *   BI8_PRE_SILU_MUL  y = cast(cast(x / (1 + exp(-x))) * x2)                     x2 [M,K] of x_dtype with x's row stride;
 *                     the two roundings of `F.silu(x) * x2` run as two kernels. */
#define BI8_PRE_NONE 0
#define BI8_PRE_RMSNORM 1
#define BI8_PRE_SILU_MUL 2
BI8_API int bi8_quantize_rowwise_pre(int op, const void* x, const void* x2, int x_dtype, int64_t ldx, const void* weight,
                             float eps, int8_t* q, float* scales, int64_t M, int64_t K, int block, void* stream);
/* bi8_gemm_dequant_fused_quant with that step in front of its quantizer and an optional residual behind its result:
 *   C = cast(acc) (+ cast(bias)) (+ residual), every addition in the output type (a layer's `x + proj(...)`).
 * residual [M,N] of out_dtype, row stride ldr, NULL for none.  For M <= 64 (N a multiple of 4, K of 16, workspace given) the
 * quantizer kernel of `op` takes the decode quantizer's place in front of the weight-streaming GEMM (same overlap), and
 * without bias the residual is added by the kernel that writes C; on that path, and only there, C may be the residual
 * itself (a residual stream updated in place; any other overlap of the two is BI8_ERR_SHAPE, the same tensor on another
 * path BI8_ERR_ALIGN).  Other shapes run quantizer, GEMM and one elementwise kernel back to back.  xq / sx are required
 * scratch. */
BI8_API int bi8_gemm_dequant_fused_pre(int op, const void* x, const void* x2, int x_dtype, int64_t ldx, const void* norm_weight,
                               float eps, int8_t* xq, float* sx, const int8_t* Wq, int64_t ldw, const float* sW,
                               const void* bias, int bias_dtype, const void* residual, int64_t ldr, void* C, int64_t ldc,
                               int out_dtype, int64_t M, int64_t N, int64_t K, int block, void* workspace,
                               size_t workspace_bytes, int flags, void* stream);

/* Model-side helper for a decode step (no counterpart in the reference, which has no model code): rotary embedding of q and
 * k and the append of k and v to the caches, in one launch, for the tensors a fused q/k/v projection leaves.
 *   qkv      [B, 3, H, D] of dtype (bf16 or fp16), contiguous: q, k, v of one new token per sequence
 *   cis      [D/2] pairs (cos, sin) fp32 of this step's position: (x0 + i x1) * (cos + i sin) per (even, odd) feature pair,
 *            fp32 products and sums each rounded on their own, result rounded to dtype
 *   pos      device address of the position (int64): row of the caches that receives k and v; read by the kernel, so the
 *            launch can be replayed from a CUDA graph while the position advances; outside [0, max_len) nothing is written
 *   q_out    [B, H, D]; kcache, vcache [B, H, max_len, D], all of dtype, contiguous. */
BI8_API int bi8_rope_cache_append(const void* qkv, int dtype, const float* cis, const long long* pos, void* q_out, void* kcache,
                          void* vcache, int64_t B, int64_t H, int64_t D, int64_t max_len, void* stream);

/* Capture sequence number of `stream` if it is being captured into a CUDA graph, 0 otherwise (no counterpart in the
 * reference).  A host layer that caches workspaces uses it to give every captured graph a scratch buffer of its own:
 * an address baked into a graph must not be shared with another graph that may be replayed on a different stream. */
BI8_API int bi8_stream_capture_id(void* stream, unsigned long long* id);

/* Diagnostic twin of bi8_gemm_dequant (no counterpart in the reference) that exercises the bounded waits of the general
 * tensor-core kernel without hanging anything.  The kernel's mbarrier waits give up after about wait_limit_us
 * microseconds (0 = the default of about two seconds), and the producer warp of every CTA leaves out the operand copies
 * of K stage skip_stage of its first tile (-1 = none), so the MMA warp's wait for that stage runs out.  Every warp then
 * leaves its loop, the CTA frees its tensor memory and the kernel returns normally; C is unspecified.  Afterwards
 * bi8_device_status() returns BI8_ERR_TIMEOUT with detail 2 (the wait for operand tiles) and clears the status word.
 * Needs a shape the tensor-core kernel takes (16-byte aligned operand rows, block 32/64/128). */
BI8_API int bi8_gemm_wait_selftest(const int8_t* A, int64_t lda, const int8_t* Bt, int64_t ldb,
                           const float* sA, const float* sB, void* C, int64_t ldc, int out_dtype,
                           int64_t M, int64_t N, int64_t K, int block, unsigned wait_limit_us, int skip_stage, void* stream);

/* Row-parallel layers (the contraction dimension of block_linear.py:141-143 divided over ranks on block boundaries)
 * leave an fp32 partial result [M,N] on every rank; the layer's output is their sum in rank order, cast, plus bias.
 * bi8_peer_allreduce does that sum with one kernel per rank over peer-mapped memory (plain loads and stores over
 * NVLink, bounded flag waits), so that it can sit in a CUDA graph between the layer's GEMM and the next layer.
 *   peer_bufs[r]  device address, valid on THIS device, of rank r's exchange buffer: bi8_peer_allreduce_buffer_bytes(world,
 *                 capacity) bytes, 16-byte aligned, zero-filled once before the first call, mapped by every rank (for
 *                 example a torch.distributed._symmetric_memory allocation, or CUDA IPC handles).  peer_bufs[rank] is
 *                 this rank's own buffer.  capacity = fp32 values per rank and reduction, a multiple of 1024, >= M*N.
 *   partial       this rank's [M,N] fp32 partial result (contiguous, 16-byte aligned), N a multiple of 4.
 *   out           [M,N] contiguous of out_dtype = cast(sum over ranks in ascending order) (+ cast(bias) in the output type):
 *                 bit-identical on all ranks.
 *   wait_limit_us how long a CTA waits for the other ranks' flags (0 = one second); when it runs out the kernel records
 *                 BI8_ERR_TIMEOUT (bi8_device_status) and returns without writing its part of `out`.
 *   bias          [N] of bias_dtype, or NULL.  With BI8_ADDEND_FULL or-ed into bias_dtype the operand is instead a
 *                 contiguous [M,N] tensor added element by element in the output type: the residual of a transformer
 *                 layer's `x + proj(...)` (it may be `out` itself).  These two entry points alone accept the flag.
 * Every rank must call it the same number of times with the same M and N.  world <= 8. */
#define BI8_ADDEND_FULL 0x100
BI8_API size_t bi8_peer_allreduce_buffer_bytes(int world, int64_t capacity);
BI8_API int bi8_peer_allreduce(void* const* peer_bufs, int rank, int world, int64_t capacity, const float* partial,
                       int64_t M, int64_t N, const void* bias, int bias_dtype, void* out, int out_dtype,
                       unsigned wait_limit_us, void* stream);

/* The same sum for prefill-sized results, where pushing every rank's whole partial result to every rank would move `world`
 * times the bytes: every rank owns one chunk in `world` of the result, loads that chunk of every rank's partial result over
 * NVLink, adds in rank order, casts, adds bias or addend, and stores the chunk into every rank's output (reduce-scatter by
 * peer loads, all-gather by peer stores, in one kernel per rank; (world-1)/world of the fp32 result in and of the cast
 * result out per rank).  The partial results and the outputs live INSIDE the peer-mapped buffers:
 *   peer_bufs[r]  rank r's buffer, bi8_peer_allreduce_large_buffer_bytes(world, capacity) bytes, zero-filled once, mapped
 *                 by every rank.  At byte offset bi8_peer_allreduce_large_partial_offset() lies the rank's partial region
 *                 ([M,N] fp32, contiguous: hand it to the GEMM as its output C), at
 *                 bi8_peer_allreduce_large_out_offset(capacity) the output region, where the call leaves [M,N] of
 *                 out_dtype, contiguous, complete on every rank when the kernel ends; it stays valid until the next call.
 * bias / bias_dtype (BI8_ADDEND_FULL for a residual, which may be the output region itself) and wait_limit_us as in
 * bi8_peer_allreduce.  The kernel waits (bounded) for the other ranks at its start and at its end. */
BI8_API size_t bi8_peer_allreduce_large_buffer_bytes(int world, int64_t capacity);
BI8_API size_t bi8_peer_allreduce_large_partial_offset(void);
BI8_API size_t bi8_peer_allreduce_large_out_offset(int64_t capacity);
BI8_API int bi8_peer_allreduce_large(void* const* peer_bufs, int rank, int world, int64_t capacity, int64_t M, int64_t N,
                             const void* bias, int bias_dtype, int out_dtype, unsigned wait_limit_us, void* stream);

/* A whole row-parallel layer in one call: quantize x [M,K] (this rank's slice of the input features), multiply with this
 * rank's weight slice Wq [N,K] / sW, and sum the ranks' fp32 partial results as bi8_peer_allreduce does.  For M <= 64
 * (decode) the kernel that adds the weight-streaming GEMM's tile parts hands its sums straight to the exchange, so the layer
 * is three launches (quantizer, GEMM, reduction over parts and ranks) with no fp32 round trip in between; other shapes run
 * bi8_gemm_dequant_fused_quant into `partial` followed by bi8_peer_allreduce.  Same results as those two calls.
 * xq [M,K] int8 and sx [ceil(K/block), M] fp32 are scratch as in bi8_gemm_dequant_fused_quant; partial [M,N] fp32 is scratch
 * (16-byte aligned); workspace as in bi8_gemm_dequant; peer_bufs .. capacity, bias, out, wait_limit_us as in
 * bi8_peer_allreduce (out [M,N] contiguous, N a multiple of 4). */
BI8_API int bi8_row_parallel_linear(const void* x, int x_dtype, int64_t ldx, int8_t* xq, float* sx, const int8_t* Wq, int64_t ldw,
                            const float* sW, float* partial, int64_t M, int64_t N, int64_t K, int block,
                            void* workspace, size_t workspace_bytes, void* const* peer_bufs, int rank, int world,
                            int64_t capacity, const void* bias, int bias_dtype, void* out, int out_dtype,
                            unsigned wait_limit_us, int flags, void* stream);
/* The same with the producer step `op` (x2, norm_weight, eps as in bi8_quantize_rowwise_pre) in front of the quantizer. */
BI8_API int bi8_row_parallel_linear_pre(int op, const void* x, const void* x2, int x_dtype, int64_t ldx, const void* norm_weight,
                                float eps, int8_t* xq, float* sx, const int8_t* Wq, int64_t ldw, const float* sW,
                                float* partial, int64_t M, int64_t N, int64_t K, int block, void* workspace,
                                size_t workspace_bytes, void* const* peer_bufs, int rank, int world, int64_t capacity,
                                const void* bias, int bias_dtype, void* out, int out_dtype, unsigned wait_limit_us, int flags,
                                void* stream);

/* Back-to-back tcgen05.mma kind::i8 issue rate of the current device: runs `iters` 128x256x32 MMAs per SM
 * with no loads or epilogue and returns the elapsed milliseconds in *ms (synchronises).  Used by the
 * benchmark to state the measured dense INT8 peak next to the nominal one. */
BI8_API int bi8_mma_peak_probe(int iters, float* ms, int* sm_count);

#ifdef __cplusplus
}
#endif
#endif /* BI8_H_ */
