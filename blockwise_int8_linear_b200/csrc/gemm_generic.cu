// CUDA-core int8 block GEMM: any strides, any block size, any alignment.
//
// Used where the tensor-core kernel does not apply (operand rows not 16-byte aligned, block sizes other
// than 32/64/128) and as an on-device cross-check.  It evaluates the accumulation in exactly the order of
// the reference kernel, triton_functions.py:120 (path inside the reference project):
//     acc += sB[j,n] * (sA[j,m] * (float(P_j) * fl32(1/127^2)))      j ascending, every step rounded to fp32
// so its fp32 results equal the CPU restatement bit for bit.
#include "bi8_common.cuh"

namespace bi8 {
namespace {

constexpr int kTile = 32;      // output tile edge
constexpr int kChunk = 32;     // K elements staged per step

template <bool PARTIALS>
__global__ void __launch_bounds__(256) gemm_generic_kernel(
    const int8_t* __restrict__ A, int64_t lda, const int8_t* __restrict__ Bt, int64_t ldb, const float* __restrict__ sA,
    const float* __restrict__ sB, const void* __restrict__ bias, int bias_dtype, void* __restrict__ C, int64_t ldc,
    int out_dtype, int32_t* __restrict__ partials, int64_t M, int64_t N, int64_t K, int B, int64_t tiles_n) {
    __shared__ __align__(16) int8_t As[kTile][kChunk + 4];
    __shared__ __align__(16) int8_t Bs[kTile][kChunk + 4];
    const int64_t m0 = (blockIdx.x / tiles_n) * kTile, n0 = (blockIdx.x % tiles_n) * kTile;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;     // thread -> outputs (2*ty + {0,1}, 2*tx + {0,1})
    const int64_t nb = (K + B - 1) / B;
    const float divf = 1.0f / (127.0f * 127.0f);
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int64_t j = 0; j < nb; ++j) {
        const int64_t lo = j * B, hi = (lo + B < K) ? lo + B : K;
        int32_t P[2][2] = {{0, 0}, {0, 0}};
        for (int64_t k0 = lo; k0 < hi; k0 += kChunk) {
            __syncthreads();
            for (int e = threadIdx.x; e < kTile * kChunk; e += 256) {
                const int r = e / kChunk, kk = e % kChunk;
                const int64_t k = k0 + kk;
                As[r][kk] = (m0 + r < M && k < hi) ? A[(m0 + r) * lda + k] : (int8_t)0;
                Bs[r][kk] = (n0 + r < N && k < hi) ? Bt[(n0 + r) * ldb + k] : (int8_t)0;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < kChunk; kk += 4) {
                int a[2], b[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    a[u] = *reinterpret_cast<const int*>(&As[2 * ty + u][kk]);
                    b[u] = *reinterpret_cast<const int*>(&Bs[2 * tx + u][kk]);
                }
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int v = 0; v < 2; ++v) P[u][v] = __dp4a(a[u], b[v], P[u][v]);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                const int64_t m = m0 + 2 * ty + u, n = n0 + 2 * tx + v;
                if (m < M && n < N) {
                    if (PARTIALS) {
                        partials[(j * M + m) * N + n] = P[u][v];
                    } else {
                        const float t0 = __fmul_rn((float)P[u][v], divf);
                        const float t1 = __fmul_rn(sA[j * M + m], t0);
                        const float t2 = __fmul_rn(sB[j * N + n], t1);
                        acc[u][v] = __fadd_rn(acc[u][v], t2);
                    }
                }
            }
    }
    if (PARTIALS) return;
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            const int64_t m = m0 + 2 * ty + u, n = n0 + 2 * tx + v;
            if (m >= M || n >= N) continue;
            float bv = 0.0f;
            const bool hb = bias != nullptr;
            if (hb) {
                if (bias_dtype == BI8_BF16) bv = __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
                else if (bias_dtype == BI8_F16) bv = __half2float(static_cast<const __half*>(bias)[n]);
                else bv = static_cast<const float*>(bias)[n];
            }
            // cast first, then add the bias in the output type (triton_functions.py:125-131)
            if (out_dtype == BI8_F32) {
                float c = acc[u][v];
                if (hb) c = __fadd_rn(c, bv);
                static_cast<float*>(C)[m * ldc + n] = c;
            } else if (out_dtype == BI8_BF16) {
                __nv_bfloat16 c = __float2bfloat16_rn(acc[u][v]);
                if (hb) c = __float2bfloat16_rn(__fadd_rn(__bfloat162float(c), __bfloat162float(__float2bfloat16_rn(bv))));
                static_cast<__nv_bfloat16*>(C)[m * ldc + n] = c;
            } else {
                __half c = __float2half_rn(acc[u][v]);
                if (hb) c = __float2half_rn(__fadd_rn(__half2float(c), __half2float(__float2half_rn(bv))));
                static_cast<__half*>(C)[m * ldc + n] = c;
            }
        }
}

}  // namespace

int launch_gemm_generic(const GemmArgs& g, cudaStream_t st) {
    const int64_t tiles_m = (g.M + kTile - 1) / kTile, tiles_n = (g.N + kTile - 1) / kTile;
    if (tiles_m * tiles_n >= (1ll << 31)) return fail(BI8_ERR_SHAPE, "generic GEMM: too many tiles");
    const unsigned grid = (unsigned)(tiles_m * tiles_n);
    if (g.partials)
        gemm_generic_kernel<true><<<grid, 256, 0, st>>>(g.A, g.lda, g.Bt, g.ldb, g.sA, g.sB, g.bias, g.bias_dtype, g.C,
                                                       g.ldc, g.out_dtype, g.partials, g.M, g.N, g.K, g.block, tiles_n);
    else
        gemm_generic_kernel<false><<<grid, 256, 0, st>>>(g.A, g.lda, g.Bt, g.ldb, g.sA, g.sB, g.bias, g.bias_dtype, g.C,
                                                        g.ldc, g.out_dtype, g.partials, g.M, g.N, g.K, g.block, tiles_n);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

}  // namespace bi8
