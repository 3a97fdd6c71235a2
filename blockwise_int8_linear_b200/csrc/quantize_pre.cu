// Row-wise block quantizers with the elementwise step that produces their input fused in front.
//
// In a transformer layer the input of every quantized projection comes out of a short elementwise step: the
// normalisation in front of q/k/v and gate/up, the gated activation in front of the down projection.  Run as separate
// kernels these write a [M, K] tensor in the activation type that the quantizer (triton_functions.py:411-423 in the
// reference, one program per row) reads back at once.  The kernels here compute that tensor in registers, round every
// value to the activation type exactly as the separate kernel would have stored it, and quantize it with the same
// arithmetic as the stand-alone quantizer (quant_math.cuh), so that the int8 values and scales are those of
// quantize_block_rowwise applied to the rounded tensor.
//
//   BI8_PRE_RMSNORM   y = cast(x * rsqrt(sum(x^2) / K + eps) [* weight])        one rounding, fp32 arithmetic
//   BI8_PRE_SILU_MUL  y = cast(cast(x / (1 + exp(-x))) * x2)                    two roundings: silu(x), then the product
//
// Both release their programmatic dependents at once (the decode GEMM launched behind them sets up and streams its first
// weights while they run; it waits for their completion before it reads the activations).  For decode-sized batches they
// are themselves launched as programmatic dependents of whatever precedes them in the stream, wait for it first thing,
// and release their own dependents only then: behind one of this library's reduction kernels (the previous layer's)
// they are resident before that kernel has finished.
#include "bi8_common.cuh"
#include "quant_math.cuh"

#include <cstring>

namespace bi8 {
namespace {

constexpr int kPreThreads = 256;
constexpr int kPreHold = 4;        // 8-element units of a row a thread keeps in registers between the two passes

// eight consecutive elements of a row, beginning at element `k` of `K`; elements from K on read as zero
__device__ __forceinline__ void load8(float* f, const void* base, int64_t row_off, int k, int K, int dt, bool vec) {
    const int esz = dt == BI8_F32 ? 4 : 2;
    const unsigned char* src = static_cast<const unsigned char*>(base) + (row_off + k) * esz;
    if (vec && k + 8 <= K) {
        const uint4 a = ld_nc_v4(src);
        if (dt == BI8_F32) {
            const uint4 b = ld_nc_v4(src + 16);
            f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
            f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
        } else {
            const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                if (dt == BI8_BF16) {
                    f[2 * h] = bf16lo(w4[h]);
                    f[2 * h + 1] = bf16hi(w4[h]);
                } else {
                    const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&w4[h]));
                    f[2 * h] = t2.x;
                    f[2 * h + 1] = t2.y;
                }
            }
        }
        return;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        float v = 0.0f;
        if (k + e < K) {
            if (dt == BI8_F32) v = reinterpret_cast<const float*>(src)[e];
            else if (dt == BI8_BF16) v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[e]);
            else v = __half2float(reinterpret_cast<const __half*>(src)[e]);
        }
        f[e] = v;
    }
}

// the same eight elements of a 16-bit type as four packed words (what a thread keeps between the two passes of a row)
__device__ __forceinline__ void load_raw8(uint32_t* w, const void* base, int64_t row_off, int k, int K, bool vec) {
    const unsigned char* src = static_cast<const unsigned char*>(base) + (row_off + k) * 2;
    if (vec && k + 8 <= K) {
        const uint4 a = ld_nc_v4(src);
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
        return;
    }
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        const uint32_t lo = k + 2 * h < K ? reinterpret_cast<const unsigned short*>(src)[2 * h] : 0u;
        const uint32_t hi = k + 2 * h + 1 < K ? reinterpret_cast<const unsigned short*>(src)[2 * h + 1] : 0u;
        w[h] = lo | (hi << 16);
    }
}

__device__ __forceinline__ void unpack8(float* f, const uint32_t* w, int dt) {
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        if (dt == BI8_BF16) {
            f[2 * h] = bf16lo(w[h]);
            f[2 * h + 1] = bf16hi(w[h]);
        } else {
            const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&w[h]));
            f[2 * h] = t2.x;
            f[2 * h + 1] = t2.y;
        }
    }
}

// the value a kernel storing `v` in the activation type would have left in memory
__device__ __forceinline__ float round_to(float v, int dt) {
    if (dt == BI8_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    if (dt == BI8_F16) return __half2float(__float2half_rn(v));
    return v;
}

// Quantizes the eight values of a unit whose block's other units sit in the neighbouring lanes (LPB lanes per block)
// and stores them; all 32 lanes of the warp must call it.
template <int QB>
__device__ __forceinline__ void quantize_unit(const float* y, bool valid, bool short_mantissa, int8_t* q, float* sx, int m, int k,
                                              int M, int K, bool vec) {
    constexpr int LPB = QB / 8;
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(y[e]));
#pragma unroll
    for (int off = 1; off < LPB; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    BlockQ bq;
    bq.set(amax, short_mantissa);
    // the exact-division shortcut on packed pairs when every block of the warp qualifies (a lane without a unit does not
    // count); else the scalar form with its per-block choice
    const bool warp_fast = __all_sync(0xffffffffu, bq.fast || !valid);
    if (!valid) return;
    uint32_t b[8];
    if (warp_fast) {
        const uint64_t r2 = f2_pack(bq.rcp, bq.rcp), ns2 = f2_pack(-amax, -amax);
        const uint64_t c127 = f2_pack(127.0f, 127.0f), cmagic = f2_pack(kMagic, kMagic), cone = f2_pack(1.0f, 1.0f);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const uint64_t v2 = f2_pack(y[2 * h], y[2 * h + 1]);
            const uint64_t q0 = f2_mul(v2, r2);
            const uint64_t e = f2_fma(ns2, q0, v2);
            const uint64_t yq = f2_fma(e, r2, q0);
            f2_bits(f2_fma(f2_mul(c127, yq), cone, cmagic), b[2 * h], b[2 * h + 1]);
        }
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) b[e] = bq.q(y[e]);
    }
    const uint32_t lo = pack4(b[0], b[1], b[2], b[3]);
    const uint32_t hi = pack4(b[4], b[5], b[6], b[7]);
    int8_t* dst = q + (int64_t)m * K + k;
    if (vec && k + 8 <= K) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (k + e < K) dst[e] = (int8_t)(((e < 4 ? lo : hi) >> (8 * (e & 3))) & 0xffu);
    }
    if (((k / 8) % LPB) == 0) sx[(int64_t)(k / QB) * M + m] = amax;
}

// One CTA per row.  Pass 1: the row's sum of squares (a thread's units in ascending order, lanes by butterfly, warps in
// ascending order: the same bits on every launch with the same THREADS, which the launcher picks from M and K).  Pass 2: normalise, round, quantize.  Rows of up
// to kPreHold * THREADS * 8 elements stay in registers between the passes; longer rows are read again.  THREADS = 128
// for rows of up to 4096 elements: a row is in flight for a load latency plus a reduction, so what bounds a large
// batch is the number of rows resident per SM (ten CTAs of 128 threads against four of 256).
template <int QB, int THREADS, int DT>
__global__ void __launch_bounds__(THREADS, THREADS == 128 ? 10 : 4) rmsnorm_quantize_kernel(const void* __restrict__ x, int64_t ldx,
                                                                       const void* __restrict__ weight, float eps,
                                                                       int8_t* __restrict__ q, float* __restrict__ sx, int M, int K,
                                                                       int nb, int vec_in, int vec_out) {
    asm volatile("griddepcontrol.wait;" ::: "memory");           // a no-op unless launched as a programmatic dependent
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int LPB = QB / 8;
    constexpr int dt = DT;                                        // the element type is a template parameter: no per-element tests
    __shared__ float warp_sum[THREADS / 32];
    const int m = blockIdx.x, tid = threadIdx.x;
    const int upr = nb * LPB;                                   // units per row, padded to whole blocks
    // 16-bit rows that fit are kept as packed words (four registers per unit); fp32 rows and longer ones are read again
    const bool hold = dt != BI8_F32 && upr <= kPreHold * THREADS;
    const int64_t row_off = (int64_t)m * ldx;
    uint32_t raw[kPreHold][4];
    float ss = 0.0f;
    if (hold) {
#pragma unroll
        for (int i = 0; i < kPreHold; ++i) {
            const int k = (i * THREADS + tid) * 8;
            if (k < K) load_raw8(raw[i], x, row_off, k, K, vec_in != 0);
            else raw[i][0] = raw[i][1] = raw[i][2] = raw[i][3] = 0u;
        }
#pragma unroll
        for (int i = 0; i < kPreHold; ++i) {
            float t[8];
            unpack8(t, raw[i], dt);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = __fmaf_rn(t[e], t[e], ss);
        }
    } else {
        for (int u = tid; u < upr; u += THREADS) {
            const int k = u * 8;
            if (k >= K) break;
            float t[8];
            load8(t, x, row_off, k, K, dt, vec_in != 0);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = __fmaf_rn(t[e], t[e], ss);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((tid & 31) == 0) warp_sum[tid >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) total += warp_sum[w];
    const float rstd = rsqrtf(__fadd_rn(__fdiv_rn(total, (float)K), eps));
    const bool short_mantissa = dt != BI8_F32;
    // normalises, rounds and quantizes the unit whose elements are in y (all lanes of a warp call it together)
    auto finish_unit = [&](float* y, int k, bool valid) {
        if (valid) {
            float w8[8];
            if (weight) load8(w8, weight, 0, k, K, dt, vec_in != 0);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float v = __fmul_rn(y[e], rstd);
                if (weight) v = __fmul_rn(v, w8[e]);
                y[e] = round_to(v, dt);
            }
        }
        quantize_unit<QB>(y, valid, short_mantissa, q, sx, m, k, M, K, vec_out != 0);
    };
    if (hold) {
#pragma unroll
        for (int i = 0; i < kPreHold; ++i) {
            if (i * THREADS < upr) {                            // the same for all threads of the CTA
                const int u = i * THREADS + tid, k = u * 8;
                float y[8];
                unpack8(y, raw[i], dt);
                finish_unit(y, k, u < upr && k < K);
            }
        }
    } else {
        for (int i = 0; i * THREADS < upr; ++i) {
            const int u = i * THREADS + tid, k = u * 8;
            const bool valid = u < upr && k < K;
            float y[8];
            if (valid) {
                load8(y, x, row_off, k, K, dt, vec_in != 0);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = 0.0f;
            }
            finish_unit(y, k, valid);
        }
    }
}

// One thread per unit of eight elements, as in the decode quantizer.
template <int QB, int DT>
__global__ void __launch_bounds__(kPreThreads) silu_mul_quantize_kernel(const void* __restrict__ gate, const void* __restrict__ up,
                                                                        int64_t ldx, int8_t* __restrict__ q,
                                                                        float* __restrict__ sx, int M, int K, int nb, int vec_in,
                                                                        int vec_out) {
    asm volatile("griddepcontrol.wait;" ::: "memory");           // a no-op unless launched as a programmatic dependent
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int LPB = QB / 8;
    constexpr int dt = DT;
    const int upr = nb * LPB;
    const int64_t u = (int64_t)blockIdx.x * kPreThreads + threadIdx.x;
    const int m = (int)(u / upr), k = (int)(u % upr) * 8;
    const bool valid = m < M && k < K;
    float y[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = 0.0f;
    if (valid) {
        float g[8], v[8];
        load8(g, gate, (int64_t)m * ldx, k, K, dt, vec_in != 0);
        load8(v, up, (int64_t)m * ldx, k, K, dt, vec_in != 0);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float s = round_to(__fdiv_rn(g[e], __fadd_rn(1.0f, expf(-g[e]))), dt);
            y[e] = round_to(__fmul_rn(s, v[e]), dt);
        }
    }
    quantize_unit<QB>(y, valid, dt != BI8_F32, q, sx, m, k, M, K, vec_out != 0);
}

// C[m, n] = cast(C[m, n] + R[m, n]): the addition a layer's `x + proj(...)` performs in the activation type
__global__ void __launch_bounds__(kPreThreads) residual_add_kernel(void* C, int64_t ldc, const void* R, int64_t ldr, int dt, int64_t M,
                                                                   int64_t N) {
    const int64_t i = (int64_t)blockIdx.x * kPreThreads + threadIdx.x;
    if (i >= M * N) return;
    const int64_t m = i / N, n = i % N, c = m * ldc + n, r = m * ldr + n;
    if (dt == BI8_F32) {
        static_cast<float*>(C)[c] = __fadd_rn(static_cast<float*>(C)[c], static_cast<const float*>(R)[r]);
    } else if (dt == BI8_BF16) {
        __nv_bfloat16* cp = static_cast<__nv_bfloat16*>(C);
        cp[c] = __float2bfloat16_rn(__fadd_rn(__bfloat162float(cp[c]), __bfloat162float(static_cast<const __nv_bfloat16*>(R)[r])));
    } else {
        __half* cp = static_cast<__half*>(C);
        cp[c] = __float2half_rn(__fadd_rn(__half2float(cp[c]), __half2float(static_cast<const __half*>(R)[r])));
    }
}

}  // namespace

int launch_residual_add(void* C, int64_t ldc, const void* R, int64_t ldr, int dt, int64_t M, int64_t N, cudaStream_t st) {
    if (M <= 0 || N <= 0) return BI8_OK;
    const int64_t blocks = (M * N + kPreThreads - 1) / kPreThreads;
    if (blocks > 0x7fffffff) return fail(BI8_ERR_LIMIT, "residual add: more than 2^31 blocks");
    residual_add_kernel<<<(unsigned)blocks, kPreThreads, 0, st>>>(C, ldc, R, ldr, dt, M, N);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

int launch_quantize_pre(int op, const void* x, const void* x2, int dt, int64_t ldx, const void* weight, float eps, int8_t* q, float* sx,
                        int64_t M, int64_t K, int block, cudaStream_t st) {
    if (M == 0 || K == 0) return BI8_OK;
    if (M > 0x7fffffff || K > 0x3fffffff) return fail(BI8_ERR_LIMIT, "quantize_pre: M or K too large");
    const int esz = dt == BI8_F32 ? 4 : 2;
    const int nb = (int)((K + block - 1) / block);
    const bool rows16 = (ldx * esz) % 16 == 0 && K % 8 == 0;
    const int vec_in = rows16 && aligned(x, 16) && (!x2 || aligned(x2, 16)) && (!weight || aligned(weight, 16));
    const int vec_out = K % 8 == 0 && aligned(q, 8);
    if (op == BI8_PRE_NONE) return launch_quantize_rowwise(x, dt, ldx, q, sx, M, K, block, st);
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = M <= 64 ? 1 : 0;       // decode: resident while the predecessor finishes (the kernels wait for it themselves)
    const int Mi = (int)M, Ki = (int)K;
    if (op == BI8_PRE_RMSNORM) {
        // 128 threads per row where the row fits their registers and there are rows enough to fill the SMs ten deep; a
        // handful of decode rows finish sooner with 256 threads each
        const bool narrow = (int64_t)nb * (block / 8) <= kPreHold * 128 && M > 1024;
        cfg.gridDim = dim3((unsigned)M);
        cfg.blockDim = dim3(narrow ? 128 : 256);
#define BI8_PRE_RMS_T(QB, T)                                                                                                          \
    do {                                                                                                                             \
        if (dt == BI8_BF16) BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, rmsnorm_quantize_kernel<QB, T, BI8_BF16>, x, ldx, weight, eps, q, sx, Mi, Ki, nb, vec_in, vec_out)); \
        else if (dt == BI8_F16) BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, rmsnorm_quantize_kernel<QB, T, BI8_F16>, x, ldx, weight, eps, q, sx, Mi, Ki, nb, vec_in, vec_out)); \
        else BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, rmsnorm_quantize_kernel<QB, T, BI8_F32>, x, ldx, weight, eps, q, sx, Mi, Ki, nb, vec_in, vec_out)); \
    } while (0)
#define BI8_PRE_RMS(QB)                                                                                                              \
    if (narrow) BI8_PRE_RMS_T(QB, 128);                                                                                              \
    else BI8_PRE_RMS_T(QB, 256)
        switch (block) {
            case 32: BI8_PRE_RMS(32); break;
            case 64: BI8_PRE_RMS(64); break;
            case 128: BI8_PRE_RMS(128); break;
            default: return fail(BI8_ERR_BLOCK, "quantize_pre supports block 32, 64, 128 (got %d)", block);
        }
#undef BI8_PRE_RMS
#undef BI8_PRE_RMS_T
    } else if (op == BI8_PRE_SILU_MUL) {
        if (!x2) return fail(BI8_ERR_NULL, "quantize_pre: the gated activation needs its second operand");
        const int64_t units = M * nb * (block / 8);
        cfg.gridDim = dim3((unsigned)((units + kPreThreads - 1) / kPreThreads));
        cfg.blockDim = dim3(kPreThreads);
#define BI8_PRE_SILU(QB)                                                                                                             \
    do {                                                                                                                             \
        if (dt == BI8_BF16) BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, silu_mul_quantize_kernel<QB, BI8_BF16>, x, x2, ldx, q, sx, Mi, Ki, nb, vec_in, vec_out)); \
        else if (dt == BI8_F16) BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, silu_mul_quantize_kernel<QB, BI8_F16>, x, x2, ldx, q, sx, Mi, Ki, nb, vec_in, vec_out)); \
        else BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, silu_mul_quantize_kernel<QB, BI8_F32>, x, x2, ldx, q, sx, Mi, Ki, nb, vec_in, vec_out)); \
    } while (0)
        switch (block) {
            case 32: BI8_PRE_SILU(32); break;
            case 64: BI8_PRE_SILU(64); break;
            case 128: BI8_PRE_SILU(128); break;
            default: return fail(BI8_ERR_BLOCK, "quantize_pre supports block 32, 64, 128 (got %d)", block);
        }
#undef BI8_PRE_SILU
    } else {
        return fail(BI8_ERR_SHAPE, "quantize_pre: unknown operation code %d", op);
    }
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

}  // namespace bi8
