// Weight-streaming int8 block GEMM for very small M (decode: M <= 16), on the CUDA cores.
//
// Same semantics as the tensor-core kernel (reference kernel triton_functions.py:69-139): exact int32 block partial
// sums, every term evaluated in the reference's order sB*(sA*(float(P)*fl32(1/127^2))), fp32 accumulation.  Only the order
// in which the terms of different blocks are added differs (each lane adds the blocks it owns, then a fixed butterfly over
// the lanes), which is within the tolerance stated for the tensor-core kernel and deterministic.
//
// For M <= 8 the work is 2*M*N*K <= 16*N*K integer operations against N*K bytes of weights: the kernel is bound by reading
// the weights once from HBM, so it is organised around that stream:
//   * a CTA first copies the quantized activations (M x K int8, at most 8 rows) and their scales into shared memory; the
//     64-byte chunks of a row are stored 80 bytes apart, which makes the 16-byte reads of 32 lanes bank-conflict free;
//   * a warp owns pairs of consecutive weight rows; in one pass lane l handles the 64-byte chunk l of each row (a warp reads
//     2 KB contiguous per row, as full 32-byte sectors), i.e. whole quantisation blocks (one block of 64, two of 32, half of
//     one of 128), so no cross-lane traffic is needed until the final sum;
//   * the (row pair, pass) items of a warp form one sequence and the weights of item i+1 are loaded before item i is
//     computed; the first item's loads are issued before the activations are staged, so the HBM latency of the first
//     access overlaps the prologue;
//   * per chunk and activation row: 16 dp4a per weight row, then the block scales.
// Larger M (9..16) runs the kernel once per group of 8 activation rows; the second pass finds the weights in L2.
#include "bi8_common.cuh"

namespace bi8 {
namespace {

constexpr int kMT = 8;            // activation rows per launch
constexpr int kR = 2;             // weight rows per warp and work item
constexpr int kWarps = 8;
constexpr int kChunk = 64;        // K bytes per lane and pass
constexpr int kChunkPitch = 80;   // shared-memory distance of consecutive chunks (bank-conflict-free 16-byte reads)

__device__ __forceinline__ void ld_nc_v8(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}

// SUB = min(block, 64): quantisation sub-blocks inside one 64-byte chunk share the chunk; for block 128 two chunks share
// one scale.
template <int QB>
__global__ void __launch_bounds__(kWarps * 32, 2) gemm_smallm_kernel(
    const int8_t* __restrict__ A, int64_t lda, const int8_t* __restrict__ Bt, int64_t ldb, const float* __restrict__ sA,
    const float* __restrict__ sB, const void* __restrict__ bias, int bias_dtype, void* __restrict__ C, int64_t ldc,
    int out_dtype, int m_base, int M, int N, int K, int nb, int chunks) {
    constexpr int SUB = QB < kChunk ? QB : kChunk;       // elements per sub-block inside a chunk
    constexpr int NSUB = kChunk / SUB;                    // sub-blocks per chunk (1 or 2)
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* xs = smem;                                         // [kMT][chunks * kChunkPitch]
    const int x_pitch = chunks * kChunkPitch;
    float* sxs = reinterpret_cast<float*>(smem + (size_t)kMT * x_pitch);   // [nb][kMT]
    const int m_count = (M - m_base) < kMT ? (M - m_base) : kMT;

    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * kWarps + (threadIdx.x >> 5), nw = gridDim.x * kWarps;
    const float divf = 1.0f / (127.0f * 127.0f);
    const int groups = (N + kR - 1) / kR;
    const int passes = (chunks + 31) / 32;
    // work items of this warp: item t -> (row pair g = gw + (t / passes) * nw, pass t % passes)
    const int my_groups = gw < groups ? (groups - gw + nw - 1) / nw : 0;
    const int items = my_groups * passes;

    auto load_w = [&](int t, uint32_t (&w)[kR][16], float (&sw)[NSUB][kR]) {
        const int g = gw + (t / passes) * nw, p = t % passes;
        const int n0 = g * kR, chunk = p * 32 + lane, k0 = chunk * kChunk;
#pragma unroll
        for (int r = 0; r < kR; ++r) {
            const int n = n0 + r;
            if (n < N && chunk < chunks && k0 + kChunk <= K) {
                const int8_t* src = Bt + (int64_t)n * ldb + k0;
                ld_nc_v8(src, *reinterpret_cast<uint32_t(*)[8]>(&w[r][0]));
                ld_nc_v8(src + 32, *reinterpret_cast<uint32_t(*)[8]>(&w[r][8]));
            } else {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (n < N && chunk < chunks && k0 + q4 * 16 < K) v = ld_nc_v4(Bt + (int64_t)n * ldb + k0 + q4 * 16);
                    w[r][q4 * 4] = v.x; w[r][q4 * 4 + 1] = v.y; w[r][q4 * 4 + 2] = v.z; w[r][q4 * 4 + 3] = v.w;
                }
            }
        }
#pragma unroll
        for (int sb = 0; sb < NSUB; ++sb) {
            const int j = (k0 + sb * SUB) / QB;
#pragma unroll
            for (int r = 0; r < kR; ++r)
                sw[sb][r] = (chunk < chunks && j < nb && n0 + r < N) ? __ldg(sB + (int64_t)j * N + n0 + r) : 0.0f;
        }
    };

    uint32_t wa[kR][16], wb[kR][16];
    float swa[NSUB][kR], swb[NSUB][kR];
    if (items > 0) load_w(0, wa, swa);           // in flight while the activations are staged

    // stage activations (zero-filled beyond K and beyond the valid rows) and their scales; loads batched by 8
    {
        const int total = kMT * chunks * 4;
        for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * blockDim.x;
                v[u] = make_uint4(0u, 0u, 0u, 0u);
                if (i < total) {
                    const int m = i / (chunks * 4), piece = i % (chunks * 4);
                    if (m < m_count && piece * 16 < K) v[u] = ld_nc_v4(A + (int64_t)(m_base + m) * lda + piece * 16);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * blockDim.x;
                if (i < total) {
                    const int m = i / (chunks * 4), piece = i % (chunks * 4);
                    *reinterpret_cast<uint4*>(xs + (size_t)m * x_pitch + (piece / 4) * kChunkPitch + (piece % 4) * 16) = v[u];
                }
            }
        }
        for (int i = threadIdx.x; i < nb * kMT; i += blockDim.x) {
            const int j = i / kMT, m = i % kMT;
            sxs[i] = (m < m_count) ? __ldg(sA + (int64_t)j * M + m_base + m) : 0.0f;
        }
    }
    __syncthreads();

    float acc[kR][kMT];
#pragma unroll
    for (int r = 0; r < kR; ++r)
#pragma unroll
        for (int m = 0; m < kMT; ++m) acc[r][m] = 0.0f;

    auto compute = [&](int t, const uint32_t (&w)[kR][16], const float (&sw)[NSUB][kR]) {
        const int p = t % passes;
        const int chunk = p * 32 + lane, k0 = chunk * kChunk;
        if (chunk < chunks) {
            const unsigned char* xrow = xs + (size_t)chunk * kChunkPitch;
#pragma unroll
            for (int m = 0; m < kMT; ++m) {
                uint32_t xv[16];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const uint4 v = *reinterpret_cast<const uint4*>(xrow + (size_t)m * x_pitch + q4 * 16);
                    xv[q4 * 4] = v.x; xv[q4 * 4 + 1] = v.y; xv[q4 * 4 + 2] = v.z; xv[q4 * 4 + 3] = v.w;
                }
#pragma unroll
                for (int sb = 0; sb < NSUB; ++sb) {
                    const int j = (k0 + sb * SUB) / QB;
                    const float sx = (j < nb) ? sxs[j * kMT + m] : 0.0f;
#pragma unroll
                    for (int r = 0; r < kR; ++r) {
                        int pacc = 0;
#pragma unroll
                        for (int q = 0; q < SUB / 4; ++q)
                            pacc = __dp4a((int)w[r][sb * (SUB / 4) + q], (int)xv[sb * (SUB / 4) + q], pacc);
                        // the reference's order for one term: sB * (sA * (float(P) * 1/127^2))
                        const float tt = __fmul_rn(sw[sb][r], __fmul_rn(sx, __fmul_rn((float)pacc, divf)));
                        acc[r][m] = __fadd_rn(acc[r][m], tt);
                    }
                }
            }
        }
        if (p == passes - 1) {
            // last pass of a row pair: fixed butterfly over the lanes, then lane (r * 8 + m) writes C[m, n0 + r]
            const int n0 = (gw + (t / passes) * nw) * kR;
            float mine = 0.0f;
#pragma unroll
            for (int r = 0; r < kR; ++r)
#pragma unroll
                for (int m = 0; m < kMT; ++m) {
                    float v = acc[r][m];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
                    if (lane == r * kMT + m) mine = v;
                    acc[r][m] = 0.0f;
                }
            const int r = lane / kMT, m = lane % kMT;
            const int n = n0 + r;
            if (r < kR && m < m_count && n < N) {
                float bv = 0.0f;
                const bool hb = bias != nullptr;
                if (hb) {
                    if (bias_dtype == BI8_BF16) bv = __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
                    else if (bias_dtype == BI8_F16) bv = __half2float(static_cast<const __half*>(bias)[n]);
                    else bv = static_cast<const float*>(bias)[n];
                }
                const int64_t o = (int64_t)(m_base + m) * ldc + n;
                if (out_dtype == BI8_F32) {
                    static_cast<float*>(C)[o] = hb ? __fadd_rn(mine, bv) : mine;
                } else if (out_dtype == BI8_BF16) {
                    __nv_bfloat16 c = __float2bfloat16_rn(mine);
                    if (hb) c = __float2bfloat16_rn(__fadd_rn(__bfloat162float(c), __bfloat162float(__float2bfloat16_rn(bv))));
                    static_cast<__nv_bfloat16*>(C)[o] = c;
                } else {
                    __half c = __float2half_rn(mine);
                    if (hb) c = __float2half_rn(__fadd_rn(__half2float(c), __half2float(__float2half_rn(bv))));
                    static_cast<__half*>(C)[o] = c;
                }
            }
        }
    };

    for (int t = 0; t < items; t += 2) {
        if (t + 1 < items) load_w(t + 1, wb, swb);
        compute(t, wa, swa);
        if (t + 1 >= items) break;
        if (t + 2 < items) load_w(t + 2, wa, swa);
        compute(t + 1, wb, swb);
    }
}

size_t smallm_smem_bytes(int64_t K, int nb) {
    const int64_t chunks = (K + kChunk - 1) / kChunk;
    return (size_t)kMT * chunks * kChunkPitch + (size_t)nb * kMT * 4;
}

}  // namespace

bool gemm_smallm_applicable(const GemmArgs& g) {
    if (g.partials != nullptr || g.M < 1 || g.M > 16) return false;
    if (g.block != 32 && g.block != 64 && g.block != 128) return false;
    if (g.K < 64 || g.K % 16 != 0 || g.K >= (1ll << 30) || g.N >= (1ll << 30)) return false;
    if (!aligned(g.A, 16) || !aligned(g.Bt, 32) || g.lda % 16 != 0 || g.ldb % 32 != 0) return false;
    const int nb = (int)((g.K + g.block - 1) / g.block);
    return smallm_smem_bytes(g.K, nb) <= 200 * 1024;
}

int launch_gemm_smallm(const GemmArgs& g, cudaStream_t st) {
    int dev = 0, sms = 0;
    BI8_CUDA_TRY(cudaGetDevice(&dev));
    BI8_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int nb = (int)((g.K + g.block - 1) / g.block);
    const int chunks = (int)((g.K + kChunk - 1) / kChunk);
    const size_t smem = smallm_smem_bytes(g.K, nb);
    const int64_t groups = (g.N + kR - 1) / kR;
    int64_t ctas = (groups + kWarps - 1) / kWarps;
    const int per_sm = smem <= 100 * 1024 ? 2 : 1;
    if (ctas > (int64_t)per_sm * sms) ctas = (int64_t)per_sm * sms;
    for (int m_base = 0; m_base < g.M; m_base += kMT) {
#define BI8_SMALLM(QB)                                                                                                  \
    {                                                                                                                   \
        static SmemOptIn opt_in;                                                                                        \
        const int orc = opt_in.ensure(gemm_smallm_kernel<QB>, smem);                                                    \
        if (orc != BI8_OK) return orc;                                                                                  \
        gemm_smallm_kernel<QB><<<(unsigned)ctas, kWarps * 32, smem, st>>>(g.A, g.lda, g.Bt, g.ldb, g.sA, g.sB, g.bias,    \
                                                                          g.bias_dtype, g.C, g.ldc, g.out_dtype, m_base,  \
                                                                          (int)g.M, (int)g.N, (int)g.K, nb, chunks);      \
    }
        if (g.block == 32) BI8_SMALLM(32)
        else if (g.block == 64) BI8_SMALLM(64)
        else BI8_SMALLM(128)
#undef BI8_SMALLM
        BI8_CUDA_TRY(cudaGetLastError());
    }
    return BI8_OK;
}

}  // namespace bi8
