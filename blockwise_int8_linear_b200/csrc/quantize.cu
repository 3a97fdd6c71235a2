// Block quantize / dequantize kernels (HBM-bound).
//
// Semantics follow the reference's kernels (paths inside the reference project):
//   quantize    triton_functions.py:382-406   scale = max|x| over the block (fp32),
//                                             q = rint(127 * (x / scale)), fp32 divide then fp32 multiply, RNE
//   dequantize  triton_functions.py:467-490   out = (scale * q) * fl32(1/127)
//   colwise     block_linear.py:93-94,100-103 transpose copy followed by the row-wise quantizer
//
// Data movement: every warp instruction of the vector kernels reads or writes one contiguous run of a
// row (32-byte or 16-byte per lane) and the block absmax is an xor-shuffle reduction inside the lanes that
// share a block.  The transposed scale tensor [K/block, rows] is written in 16-byte pieces (four rows of one
// block) by the streaming quantizer, and staged through shared memory by the tile kernels so that its
// stores (and, for dequantize, its loads) are contiguous along the row index.
#include "bi8_common.cuh"
#include "quant_math.cuh"

#include <cstdlib>

namespace bi8 {
namespace {

constexpr int kTileRows = 32;
constexpr int kThreads = 256;

__device__ __forceinline__ void ld_nc_v8(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}
__device__ __forceinline__ void st_v8(void* p, const uint32_t (&r)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                 "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }

// two packed 16-bit floats -> two fp32
template <typename T>
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi);
template <>
__device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float& lo, float& hi) {
    lo = bf16lo(w);
    hi = bf16hi(w);
}
template <>
__device__ __forceinline__ void unpack2<__half>(uint32_t w, float& lo, float& hi) {
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&w));
    lo = f.x;
    hi = f.y;
}

// ------------------------------------------------------------------------------------------------
// Row-wise quantize, vector path.  T is a 16-bit float type.  VEC elements per lane (16: one 32-byte
// load and one 16-byte store per lane; 8: 16-byte load, 8-byte store).  A CTA covers 32 rows x 32*VEC
// columns; warp w handles rows w, w+8, w+16, w+24 and issues the four loads before any arithmetic.
template <typename T, int B, int VEC>
__global__ void __launch_bounds__(kThreads) quantize_rowwise_vec_kernel(
    const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ q, float* __restrict__ s, int M, int K, int nb,
    int col_tiles) {
    constexpr int WCOLS = 32 * VEC;         // columns per warp pass
    constexpr int LPB = B / VEC;            // lanes sharing one block
    constexpr int BPT = WCOLS / B;          // blocks per tile row
    constexpr int NW = VEC / 2;             // 32-bit words loaded per lane
    static_assert(B % VEC == 0 && LPB >= 1 && LPB <= 32, "block must be a multiple of the lane vector");
    __shared__ float s_scale[BPT][kTileRows];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ct = blockIdx.x % col_tiles, rt = blockIdx.x / col_tiles;
    const int col = ct * WCOLS + lane * VEC;
    const bool col_ok = col < K;            // K % VEC == 0 on this path: a lane is all in or all out

    uint32_t raw[4][NW];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = rt * kTileRows + warp + 8 * i;
        if (col_ok && row < M) {
            const T* p = x + (int64_t)row * ldx + col;
            if constexpr (VEC == 16) {
                ld_nc_v8(p, raw[i]);
            } else {
                uint4 v = ld_nc_v4(p);
                raw[i][0] = v.x; raw[i][1] = v.y; raw[i][2] = v.z; raw[i][3] = v.w;
            }
        } else {
#pragma unroll
            for (int w = 0; w < NW; ++w) raw[i][w] = 0u;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = rt * kTileRows + warp + 8 * i;
        float v[VEC];
        float amax = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            unpack2<T>(raw[i][w], v[2 * w], v[2 * w + 1]);
            amax = fmaxf(amax, fmaxf(fabsf(v[2 * w]), fabsf(v[2 * w + 1])));
        }
#pragma unroll
        for (int off = 1; off < LPB; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        BlockQ bq;
        bq.set(amax, true);
        uint32_t out[VEC / 4];
#pragma unroll
        for (int w = 0; w < VEC / 4; ++w)
            out[w] = pack4(bq.q(v[4 * w]), bq.q(v[4 * w + 1]), bq.q(v[4 * w + 2]), bq.q(v[4 * w + 3]));
        if (col_ok && row < M) {
            int8_t* o = q + (int64_t)row * K + col;
            if constexpr (VEC == 16) {
                *reinterpret_cast<uint4*>(o) = make_uint4(out[0], out[1], out[2], out[3]);
            } else {
                *reinterpret_cast<uint2*>(o) = make_uint2(out[0], out[1]);
            }
        }
        if ((lane % LPB) == 0) s_scale[lane / LPB][warp + 8 * i] = amax;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < BPT * kTileRows; t += kThreads) {
        const int j = t / kTileRows, r = t % kTileRows;
        const int jb = ct * BPT + j, row = rt * kTileRows + r;
        if (jb < nb && row < M) s[(int64_t)jb * M + row] = s_scale[j][r];
    }
}

// Packed fp32 pairs (add/mul/fma.rn.f32x2): one instruction for two lanes of data, each lane rounded exactly
// like the scalar instruction.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack_bits(uint64_t v, uint32_t& lo, uint32_t& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// Row-wise quantize, streaming path (16-bit inputs, K % 16 == 0, 32-byte aligned rows).
// Persistent warps: a warp owns units of 4 rows x 512 columns (lane = 16 consecutive elements of a row, one
// 32-byte load and one 16-byte store per row) and keeps the loads of its NEXT unit in flight while it quantizes
// the current one, so the memory system always has 128 bytes per lane outstanding.  No shared memory and no CTA
// barrier: the lane that leads a block keeps the four row scales of its block and writes them as one 16-byte
// piece of the transposed scale tensor (s[j, m0..m0+3]).  The arithmetic is done on packed fp32 pairs.
template <typename T, int B>
__global__ void __launch_bounds__(kThreads, 2) quantize_rowwise_stream_kernel(
    const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ q, float* __restrict__ s, int M, int K, int nb,
    int col_units, int64_t total_units) {
    constexpr int LPB = B / 16;             // lanes sharing one block
    const int lane = threadIdx.x & 31;
    const int64_t gw = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const int64_t nw = (int64_t)gridDim.x * (kThreads / 32);
    // fl(127*y) and the round-to-integer step must stay two separately rounded operations.  A packed multiply
    // followed by a packed ADD was observed to come out as one fused operation (ties then round differently from
    // the reference's two-step evaluation), so the second step is written as fma(z, 1, magic): the product z*1 is
    // exact, the result is the single rounding of z + magic, and there is no multiply left to contract into it.
    const uint64_t c127 = f2_pack(127.0f, 127.0f), cmagic = f2_pack(kMagic, kMagic), cone = f2_pack(1.0f, 1.0f);
    auto round_pair = [&](uint64_t y2, uint32_t& b0, uint32_t& b1) {
        const uint64_t z = f2_mul(c127, y2);
        f2_unpack_bits(f2_fma(z, cone, cmagic), b0, b1);
    };

    auto load_unit = [&](int64_t u, uint32_t (&buf)[4][8]) {
        const int rg = (int)(u / col_units), ct = (int)(u % col_units);
        const int col = ct * 512 + lane * 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = rg * 4 + i;
            if (col < K && row < M) {
                ld_nc_v8(x + (int64_t)row * ldx + col, buf[i]);
            } else {
#pragma unroll
                for (int w = 0; w < 8; ++w) buf[i][w] = 0u;
            }
        }
    };
    auto process_unit = [&](int64_t u, const uint32_t (&buf)[4][8]) {
        const int rg = (int)(u / col_units), ct = (int)(u % col_units);
        const int col = ct * 512 + lane * 16;
        float sc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = rg * 4 + i;
            uint64_t v2[8];
            float amax = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                float lo, hi;
                unpack2<T>(buf[i][w], lo, hi);
                amax = fmaxf(amax, fmaxf(fabsf(lo), fabsf(hi)));
                v2[w] = f2_pack(lo, hi);
            }
#pragma unroll
            for (int off = 1; off < LPB; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            sc[i] = amax;
            BlockQ bq;
            bq.set(amax, true);
            uint32_t out[4];
            if (bq.fast) {
                const uint64_t r2 = f2_pack(bq.rcp, bq.rcp), ns2 = f2_pack(-amax, -amax);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    uint32_t b0, b1, b2, b3;
                    {
                        const uint64_t q0 = f2_mul(v2[2 * w], r2);
                        const uint64_t e = f2_fma(ns2, q0, v2[2 * w]);
                        const uint64_t y = f2_fma(e, r2, q0);
                        round_pair(y, b0, b1);
                    }
                    {
                        const uint64_t q0 = f2_mul(v2[2 * w + 1], r2);
                        const uint64_t e = f2_fma(ns2, q0, v2[2 * w + 1]);
                        const uint64_t y = f2_fma(e, r2, q0);
                        round_pair(y, b2, b3);
                    }
                    out[w] = pack4(b0, b1, b2, b3);
                }
            } else {
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    uint32_t a0, a1, a2, a3;
                    f2_unpack_bits(v2[2 * w], a0, a1);
                    f2_unpack_bits(v2[2 * w + 1], a2, a3);
                    out[w] = pack4(bq.q(__uint_as_float(a0)), bq.q(__uint_as_float(a1)), bq.q(__uint_as_float(a2)),
                                   bq.q(__uint_as_float(a3)));
                }
            }
            if (col < K && row < M)
                *reinterpret_cast<uint4*>(q + (int64_t)row * K + col) = make_uint4(out[0], out[1], out[2], out[3]);
        }
        if ((lane % LPB) == 0) {
            const int jb = (col / B);
            const int m0 = rg * 4;
            if (jb < nb && m0 < M) {
                float* dst = s + (int64_t)jb * M + m0;
                if (((M & 3) == 0)) {
                    *reinterpret_cast<float4*>(dst) = make_float4(sc[0], sc[1], sc[2], sc[3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (m0 + i < M) dst[i] = sc[i];
                }
            }
        }
    };

    uint32_t bufa[4][8], bufb[4][8];
    int64_t u = gw;
    if (u < total_units) load_unit(u, bufa);
    while (u < total_units) {
        const int64_t u1 = u + nw;
        if (u1 < total_units) load_unit(u1, bufb);
        process_unit(u, bufa);
        if (u1 >= total_units) break;
        const int64_t u2 = u1 + nw;
        if (u2 < total_units) load_unit(u2, bufa);
        process_unit(u1, bufb);
        u = u2;
    }
}

// Row-wise quantize, any type / block / alignment: one warp per (row, block).
// Row-wise quantize for rows that are not 16-byte aligned (row length not a multiple of 8, e.g. a 50257-wide vocabulary),
// block <= 64.  A warp takes kRagGroup consecutive blocks of one row; lane l handles elements l and l + 32 of every block, so
// all loads of the group (2-byte, coalesced) are in flight before the first absmax reduction, and the stores are runs of 32
// consecutive bytes.  Same arithmetic as every other quantizer (BlockQ).
constexpr int kRagGroup = 8;
template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_rowwise_ragged_kernel(
    const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int64_t K, int B,
    int64_t nb, int64_t groups_per_row) {
    const int lane = threadIdx.x & 31;
    const int64_t task = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (task >= M * groups_per_row) return;
    const int64_t row = task / groups_per_row, j0 = (task % groups_per_row) * kRagGroup;
    const T* xr = x + row * ldx;
    float v[kRagGroup][2];
#pragma unroll
    for (int b = 0; b < kRagGroup; ++b) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int64_t k = (j0 + b) * B + lane + 32 * e;
            const bool valid = (j0 + b) < nb && lane + 32 * e < B && k < K;
            v[b][e] = valid ? to_f32<T>(xr[k]) : 0.0f;
        }
    }
#pragma unroll
    for (int b = 0; b < kRagGroup; ++b) {
        float amax = fmaxf(fabsf(v[b][0]), fabsf(v[b][1]));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const int64_t j = j0 + b;
        if (j >= nb) continue;
        BlockQ bq;
        bq.set(amax, sizeof(T) == 2);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int64_t k = j * B + lane + 32 * e;
            if (lane + 32 * e < B && k < K) q[row * K + k] = (int8_t)(bq.q(v[b][e]) & 0xffu);
        }
        if (lane == 0) s[j * M + row] = amax;
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_rowwise_generic_kernel(
    const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int64_t K, int B,
    int64_t nb) {
    const int lane = threadIdx.x & 31;
    const int64_t task = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (task >= M * nb) return;
    const int64_t row = task / nb, j = task % nb;
    const int64_t lo = j * B, hi = (lo + B < K) ? lo + B : K;
    const T* xr = x + row * ldx;
    float amax = 0.0f;
    for (int64_t k = lo + lane; k < hi; k += 32) amax = fmaxf(amax, fabsf(to_f32<T>(xr[k])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    BlockQ bq;
    bq.set(amax, sizeof(T) == 2);
    for (int64_t k = lo + lane; k < hi; k += 32) q[row * K + k] = (int8_t)(bq.q(to_f32<T>(xr[k])) & 0xffu);
    if (lane == 0) s[j * M + row] = amax;
}

// ------------------------------------------------------------------------------------------------
// Column-wise quantize (fused transpose): x [R,C] -> q [C,R], s [ceil(R/B), C].  A CTA stages a tile of
// NBLK*B rows x 128 columns in shared memory with 16-byte row-contiguous loads; then one thread owns one
// (block, column): it reads the B values down the column once (bank-conflict free: lanes are consecutive columns),
// keeps them packed in registers, takes the absmax and quantizes.  The int8 results go back to shared memory
// transposed ([column][row], reusing the staging area), and the CTA writes them out as whole 128-byte (or longer)
// runs of the output rows.
template <typename T, int B>
__global__ void __launch_bounds__(kThreads) quantize_colwise_vec_kernel(
    const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ q, float* __restrict__ s, int R, int C, int col_tiles) {
    constexpr int TC = 128;
    constexpr int NBLK = kThreads / TC;     // blocks (along rows of x) per tile
    constexpr int TR = NBLK * B;
    constexpr int PITCH = TC + 2;           // 16-bit elements; +2 keeps column reads conflict free
    constexpr int OPITCH = TR + 16;         // bytes per output row in the transposed tile
    static_assert(TC * OPITCH <= TR * PITCH * 2, "the transposed tile reuses the staging area");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint16_t* tile = reinterpret_cast<uint16_t*>(smem_raw);

    const int ct = blockIdx.x % col_tiles, rt = blockIdx.x / col_tiles;
    const int c0 = ct * TC, r0 = rt * TR;
    // load: each row of the tile is 16 lanes x 16 bytes; all loads of a thread are issued before its first store
    constexpr int VPR = TC / 8;
    constexpr int PER_THREAD = TR * VPR / kThreads;
    {
        uint4 d[PER_THREAD];
#pragma unroll
        for (int u = 0; u < PER_THREAD; ++u) {
            const int v = threadIdx.x + u * kThreads;
            const int r = v / VPR, cv = (v % VPR) * 8;
            d[u] = make_uint4(0u, 0u, 0u, 0u);
            if (r0 + r < R && c0 + cv < C) d[u] = ld_nc_v4(x + (int64_t)(r0 + r) * ldx + c0 + cv);
        }
#pragma unroll
        for (int u = 0; u < PER_THREAD; ++u) {
            const int v = threadIdx.x + u * kThreads;
            const int r = v / VPR, cv = (v % VPR) * 8;
            uint32_t* dst = reinterpret_cast<uint32_t*>(tile + r * PITCH + cv);   // 4-byte aligned (PITCH even)
            dst[0] = d[u].x; dst[1] = d[u].y; dst[2] = d[u].z; dst[3] = d[u].w;
        }
    }
    __syncthreads();
    const int c = threadIdx.x % TC, blk = threadIdx.x / TC;
    const uint16_t* colp = tile + (blk * B) * PITCH + c;
    uint32_t packed[B / 2];                 // the column's B values, two per register
    float amax = 0.0f;
#pragma unroll
    for (int r = 0; r < B; r += 2) {
        const uint32_t lo = colp[r * PITCH], hi = colp[(r + 1) * PITCH];
        packed[r / 2] = lo | (hi << 16);
        float flo, fhi;
        unpack2<T>(packed[r / 2], flo, fhi);
        amax = fmaxf(amax, fmaxf(fabsf(flo), fabsf(fhi)));
    }
    BlockQ bq;
    bq.set(amax, true);
    uint32_t out[B / 4];
#pragma unroll
    for (int g = 0; g < B / 4; ++g) {
        float f0, f1, f2, f3;
        unpack2<T>(packed[2 * g], f0, f1);
        unpack2<T>(packed[2 * g + 1], f2, f3);
        out[g] = pack4(bq.q(f0), bq.q(f1), bq.q(f2), bq.q(f3));
    }
    const int rb = r0 + blk * B;            // first row of this block
    if (c0 + c < C && rb < R) s[(int64_t)(rb / B) * C + c0 + c] = amax;
    __syncthreads();                        // every thread has read its column: the staging area can be reused
    unsigned char* otile = smem_raw;        // [TC][OPITCH] int8, row = output row (column of x)
#pragma unroll
    for (int g = 0; g < B / 16; ++g)
        *reinterpret_cast<uint4*>(otile + c * OPITCH + blk * B + g * 16) = make_uint4(out[4 * g], out[4 * g + 1], out[4 * g + 2], out[4 * g + 3]);
    __syncthreads();
    // store: output row (c0 + cc) receives TR contiguous bytes starting at r0
    constexpr int PIECES = TR / 16;         // 16-byte pieces per output row
    const bool vec_ok = ((R & 15) == 0);
    for (int v = threadIdx.x; v < TC * PIECES; v += kThreads) {
        const int cc = v / PIECES, piece = v % PIECES;
        const int rr = r0 + piece * 16;
        if (c0 + cc >= C || rr >= R) continue;
        const uint4 d = *reinterpret_cast<const uint4*>(otile + cc * OPITCH + piece * 16);
        int8_t* o = q + (int64_t)(c0 + cc) * R + rr;
        if (vec_ok && rr + 16 <= R) {
            *reinterpret_cast<uint4*>(o) = d;
        } else {
            const uint32_t w[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (rr + u < R) o[u] = (int8_t)((w[u / 4] >> (8 * (u % 4))) & 0xffu);
        }
    }
}

// Column-wise quantize when rows of the input or of the output are not 16-byte aligned (e.g. 50257 columns).  A CTA takes
// one block of B rows x kThreads columns: thread t reads its column down the block twice (absmax, then quantize; the
// second pass hits L1/L2; consecutive threads read consecutive columns), parks the B bytes in shared memory, and the
// warps then write each output row's B bytes as runs of 32 consecutive bytes.  (With one thread storing its column byte
// by byte, every warp store touched 32 sectors.)  Dynamic shared memory: kThreads * (B + 4) bytes.
template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_colwise_ragged_kernel(
    const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ q, float* __restrict__ s, int64_t R, int64_t C, int B,
    int64_t col_tiles) {
    extern __shared__ unsigned char tile[];                 // [kThreads][B + 4]
    const int pitch = B + 4;
    const int64_t j = blockIdx.x / col_tiles, c0 = (blockIdx.x % col_tiles) * kThreads;
    const int64_t lo = j * B;
    const int rows = (int)((lo + B < R) ? B : R - lo);
    const int64_t c = c0 + threadIdx.x;
    if (c < C) {
        const T* xc = x + lo * ldx + c;
        float amax = 0.0f;
        for (int r = 0; r < rows; ++r) amax = fmaxf(amax, fabsf(to_f32<T>(xc[(int64_t)r * ldx])));
        BlockQ bq;
        bq.set(amax, sizeof(T) == 2);
        unsigned char* mine = tile + (size_t)threadIdx.x * pitch;
        for (int r = 0; r < rows; ++r) mine[r] = (unsigned char)(bq.q(to_f32<T>(xc[(int64_t)r * ldx])) & 0xffu);
        s[j * C + c] = amax;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = warp; t < kThreads; t += kThreads / 32) {
        const int64_t cc = c0 + t;
        if (cc >= C) break;
        int8_t* dst = q + cc * R + lo;
        const unsigned char* src = tile + (size_t)t * pitch;
        for (int r = lane; r < rows; r += 32) dst[r] = (int8_t)src[r];
    }
}

// Column-wise quantize, any type / block / alignment: one thread per (block, column).
template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_colwise_generic_kernel(
    const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ q, float* __restrict__ s, int64_t R, int64_t C, int B,
    int64_t nb) {
    const int64_t task = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (task >= nb * C) return;
    const int64_t j = task / C, c = task % C;
    const int64_t lo = j * B, hi = (lo + B < R) ? lo + B : R;
    float amax = 0.0f;
    for (int64_t r = lo; r < hi; ++r) amax = fmaxf(amax, fabsf(to_f32<T>(x[r * ldx + c])));
    BlockQ bq;
    bq.set(amax, sizeof(T) == 2);
    for (int64_t r = lo; r < hi; ++r) q[c * R + r] = (int8_t)(bq.q(to_f32<T>(x[r * ldx + c])) & 0xffu);
    s[j * C + c] = amax;
}

// ------------------------------------------------------------------------------------------------
// Dequantize, vector path: a lane owns 16 consecutive int8 (one 16-byte load) and writes 16 outputs.
// The CTA tile is 32 rows x 512 columns; its scales [512/B][32] are loaded row-contiguously first.
template <typename TO>
__device__ __forceinline__ void store16(TO* o, const float (&f)[16]);
template <>
__device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* o, const float (&f)[16]) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
    st_v8(o, w);
}
template <>
__device__ __forceinline__ void store16<__half>(__half* o, const float (&f)[16]) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = pack_f16x2(f[2 * i], f[2 * i + 1]);
    st_v8(o, w);
}
template <>
__device__ __forceinline__ void store16<float>(float* o, const float (&f)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4*>(o + 4 * i) = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
}

template <typename TO, int B>
__global__ void __launch_bounds__(kThreads) dequantize_rowwise_vec_kernel(
    const int8_t* __restrict__ q, const float* __restrict__ s, TO* __restrict__ out, int M, int K, int nb,
    int col_tiles) {
    constexpr int WCOLS = 512;
    constexpr int BPT = WCOLS / B;
    constexpr int LPB = B / 16;
    __shared__ float s_scale[BPT][kTileRows];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ct = blockIdx.x % col_tiles, rt = blockIdx.x / col_tiles;
    const int col = ct * WCOLS + lane * 16;
    const bool col_ok = col < K;            // K % 16 == 0 on this path

    uint4 raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = rt * kTileRows + warp + 8 * i;
        raw[i] = (col_ok && row < M) ? ld_nc_v4(q + (int64_t)row * K + col) : make_uint4(0u, 0u, 0u, 0u);
    }
    for (int t = threadIdx.x; t < BPT * kTileRows; t += kThreads) {
        const int j = t / kTileRows, r = t % kTileRows;
        const int jb = ct * BPT + j, row = rt * kTileRows + r;
        s_scale[j][r] = (jb < nb && row < M) ? s[(int64_t)jb * M + row] : 0.0f;
    }
    __syncthreads();
    const float inv127 = 1.0f / 127.0f;     // fl32(1/127), the constant the reference passes (line 499)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = rt * kTileRows + warp + 8 * i;
        if (!(col_ok && row < M)) continue;
        const float sc = s_scale[lane / LPB][warp + 8 * i];
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
        float f[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const int v = (int)(int8_t)((w[e / 4] >> (8 * (e % 4))) & 0xffu);
            f[e] = __fmul_rn(__fmul_rn(sc, (float)v), inv127);
        }
        store16<TO>(out + (int64_t)row * K + col, f);
    }
}

template <typename TO>
__device__ __forceinline__ TO from_f32(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }

template <typename TO>
__global__ void __launch_bounds__(kThreads) dequantize_rowwise_generic_kernel(
    const int8_t* __restrict__ q, const float* __restrict__ s, TO* __restrict__ out, int64_t M, int64_t K, int B) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= M * K) return;
    const int64_t m = i / K, k = i % K;
    const float inv127 = 1.0f / 127.0f;
    out[i] = from_f32<TO>(__fmul_rn(__fmul_rn(s[(k / B) * M + m], (float)q[i]), inv127));
}

bool use_v8() {
    static const bool on = (std::getenv("BI8_NO_V8") == nullptr);
    return on;
}

template <typename T>
int quantize_rowwise_t(const T* x, int64_t ldx, int8_t* q, float* s, int64_t M, int64_t K, int block, cudaStream_t st) {
    const int64_t nb = (K + block - 1) / block;
    const bool small = sizeof(T) == 2 && M < (1ll << 31) && K < (1ll << 31);
    const bool v16 = small && use_v8() && K % 16 == 0 && ldx % 16 == 0 && aligned(x, 32) && aligned(q, 16);
    const bool v8 = small && K % 8 == 0 && ldx % 8 == 0 && aligned(x, 16) && aligned(q, 8);
    const int64_t row_tiles = (M + kTileRows - 1) / kTileRows;
#define BI8_QROW(BB, VV)                                                                                   \
    do {                                                                                                   \
        const int64_t ctiles = (K + 32 * VV - 1) / (32 * VV);                                              \
        if (row_tiles * ctiles >= (1ll << 31)) break;                                                      \
        quantize_rowwise_vec_kernel<T, BB, VV><<<(unsigned)(row_tiles * ctiles), kThreads, 0, st>>>(        \
            x, ldx, q, s, (int)M, (int)K, (int)nb, (int)ctiles);                                           \
        BI8_CUDA_TRY(cudaGetLastError());                                                                  \
        return BI8_OK;                                                                                     \
    } while (0)
    if constexpr (sizeof(T) == 2) {
        if (v16 && aligned(s, 16) && (block == 32 || block == 64 || block == 128 || block == 256)) {
            int dev = 0, sms = 0;
            BI8_CUDA_TRY(cudaGetDevice(&dev));
            BI8_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            const int col_units = (int)((K + 511) / 512);
            const int64_t total = ((M + 3) / 4) * col_units;
            const int64_t warps_wanted = total;                      // one unit per warp at least
            int64_t ctas = (warps_wanted + kThreads / 32 - 1) / (kThreads / 32);
            if (ctas > 2ll * sms) ctas = 2ll * sms;                  // two resident CTAs per SM, persistent beyond that
#define BI8_QSTREAM(BB)                                                                                          \
    if (block == BB) {                                                                                           \
        quantize_rowwise_stream_kernel<T, BB><<<(unsigned)ctas, kThreads, 0, st>>>(x, ldx, q, s, (int)M, (int)K,  \
                                                                                   (int)nb, col_units, total);   \
        BI8_CUDA_TRY(cudaGetLastError());                                                                        \
        return BI8_OK;                                                                                           \
    }
            BI8_QSTREAM(32) BI8_QSTREAM(64) BI8_QSTREAM(128) BI8_QSTREAM(256)
#undef BI8_QSTREAM
        }
        if (v16) {
            if (block == 32) BI8_QROW(32, 16);
            if (block == 64) BI8_QROW(64, 16);
            if (block == 128) BI8_QROW(128, 16);
            if (block == 256) BI8_QROW(256, 16);
        }
        if (v8) {
            if (block == 32) BI8_QROW(32, 8);
            if (block == 64) BI8_QROW(64, 8);
            if (block == 128) BI8_QROW(128, 8);
            if (block == 256) BI8_QROW(256, 8);
        }
    }
#undef BI8_QROW
    if (block <= 64) {
        const int64_t gpr = (nb + kRagGroup - 1) / kRagGroup;
        const int64_t rgrid = (M * gpr + kThreads / 32 - 1) / (kThreads / 32);
        if (rgrid < (1ll << 31)) {
            quantize_rowwise_ragged_kernel<T><<<(unsigned)rgrid, kThreads, 0, st>>>(x, ldx, q, s, M, K, block, nb, gpr);
            BI8_CUDA_TRY(cudaGetLastError());
            return BI8_OK;
        }
    }
    const int64_t tasks = M * nb;
    const int64_t grid = (tasks + kThreads / 32 - 1) / (kThreads / 32);
    if (grid >= (1ll << 31)) return fail(BI8_ERR_SHAPE, "quantize_rowwise: %lld blocks exceed the grid limit", (long long)tasks);
    quantize_rowwise_generic_kernel<T><<<(unsigned)grid, kThreads, 0, st>>>(x, ldx, q, s, M, K, block, nb);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

template <typename T, int B>
int colwise_vec(const T* x, int64_t ldx, int8_t* q, float* s, int64_t R, int64_t C, cudaStream_t st) {
    constexpr int TC = 128, NBLK = kThreads / TC, TR = NBLK * B;
    const int64_t ctiles = (C + TC - 1) / TC, rtiles = (R + TR - 1) / TR;
    if (ctiles * rtiles >= (1ll << 31)) return fail(BI8_ERR_SHAPE, "quantize_colwise: grid too large");
    const size_t smem = (size_t)TR * (TC + 2) * 2;
    static SmemOptIn opt_in;                // per kernel instance; set once per device
    const int rc = opt_in.ensure(quantize_colwise_vec_kernel<T, B>, smem);
    if (rc != BI8_OK) return rc;
    quantize_colwise_vec_kernel<T, B><<<(unsigned)(ctiles * rtiles), kThreads, smem, st>>>(x, ldx, q, s, (int)R, (int)C, (int)ctiles);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

template <typename T>
int quantize_colwise_t(const T* x, int64_t ldx, int8_t* q, float* s, int64_t R, int64_t C, int block, cudaStream_t st) {
    if constexpr (sizeof(T) == 2) {
        const bool vec = R < (1ll << 31) && C < (1ll << 31) && C % 8 == 0 && ldx % 8 == 0 && aligned(x, 16) && aligned(q, 16);
        if (vec) {
            if (block == 32) return colwise_vec<T, 32>(x, ldx, q, s, R, C, st);
            if (block == 64) return colwise_vec<T, 64>(x, ldx, q, s, R, C, st);
            if (block == 128) return colwise_vec<T, 128>(x, ldx, q, s, R, C, st);
        }
    }
    const int64_t nb = (R + block - 1) / block;
    if (block <= 256) {
        const int64_t col_tiles = (C + kThreads - 1) / kThreads;
        const size_t smem = (size_t)kThreads * (block + 4);
        if (nb * col_tiles < (1ll << 31)) {
            if (smem > 48 * 1024) {
                static SmemOptIn opt_in;
                const int rc = opt_in.ensure(quantize_colwise_ragged_kernel<T>, smem);
                if (rc != BI8_OK) return rc;
            }
            quantize_colwise_ragged_kernel<T><<<(unsigned)(nb * col_tiles), kThreads, smem, st>>>(x, ldx, q, s, R, C, block, col_tiles);
            BI8_CUDA_TRY(cudaGetLastError());
            return BI8_OK;
        }
    }
    const int64_t grid = (nb * C + kThreads - 1) / kThreads;
    if (grid >= (1ll << 31)) return fail(BI8_ERR_SHAPE, "quantize_colwise: grid too large");
    quantize_colwise_generic_kernel<T><<<(unsigned)grid, kThreads, 0, st>>>(x, ldx, q, s, R, C, block, nb);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

template <typename TO>
int dequantize_t(const int8_t* q, const float* s, TO* out, int64_t M, int64_t K, int block, cudaStream_t st) {
    const int64_t nb = (K + block - 1) / block;
    const bool vec = use_v8() && M < (1ll << 31) && K < (1ll << 31) && K % 16 == 0 && aligned(q, 16) && aligned(out, 32);
    const int64_t row_tiles = (M + kTileRows - 1) / kTileRows, ctiles = (K + 511) / 512;
    if (vec && row_tiles * ctiles < (1ll << 31)) {
#define BI8_DEQ(BB)                                                                                         \
    if (block == BB) {                                                                                      \
        dequantize_rowwise_vec_kernel<TO, BB><<<(unsigned)(row_tiles * ctiles), kThreads, 0, st>>>(           \
            q, s, out, (int)M, (int)K, (int)nb, (int)ctiles);                                               \
        BI8_CUDA_TRY(cudaGetLastError());                                                                   \
        return BI8_OK;                                                                                      \
    }
        BI8_DEQ(32) BI8_DEQ(64) BI8_DEQ(128) BI8_DEQ(256)
#undef BI8_DEQ
    }
    const int64_t grid = (M * K + kThreads - 1) / kThreads;
    if (grid >= (1ll << 31)) return fail(BI8_ERR_SHAPE, "dequantize: grid too large");
    dequantize_rowwise_generic_kernel<TO><<<(unsigned)grid, kThreads, 0, st>>>(q, s, out, M, K, block);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

}  // namespace

int launch_quantize_rowwise(const void* x, int dt, int64_t ldx, int8_t* q, float* s, int64_t M, int64_t K, int block,
                            cudaStream_t st) {
    switch (dt) {
        case BI8_BF16: return quantize_rowwise_t(static_cast<const __nv_bfloat16*>(x), ldx, q, s, M, K, block, st);
        case BI8_F16: return quantize_rowwise_t(static_cast<const __half*>(x), ldx, q, s, M, K, block, st);
        case BI8_F32: return quantize_rowwise_t(static_cast<const float*>(x), ldx, q, s, M, K, block, st);
    }
    return fail(BI8_ERR_DTYPE, "quantize_rowwise: unknown dtype code %d", dt);
}

int launch_quantize_colwise(const void* x, int dt, int64_t ldx, int8_t* q, float* s, int64_t R, int64_t C, int block,
                            cudaStream_t st) {
    if (quantize_tile_applicable(x, dt, ldx, q, nullptr, R, C, block))
        return launch_quantize_tile(x, dt, ldx, q, s, nullptr, nullptr, R, C, block, st);
    switch (dt) {
        case BI8_BF16: return quantize_colwise_t(static_cast<const __nv_bfloat16*>(x), ldx, q, s, R, C, block, st);
        case BI8_F16: return quantize_colwise_t(static_cast<const __half*>(x), ldx, q, s, R, C, block, st);
        case BI8_F32: return quantize_colwise_t(static_cast<const float*>(x), ldx, q, s, R, C, block, st);
    }
    return fail(BI8_ERR_DTYPE, "quantize_colwise: unknown dtype code %d", dt);
}

int launch_dequantize_rowwise(const int8_t* q, const float* s, void* out, int dt, int64_t M, int64_t K, int block,
                              cudaStream_t st) {
    switch (dt) {
        case BI8_BF16: return dequantize_t(q, s, static_cast<__nv_bfloat16*>(out), M, K, block, st);
        case BI8_F16: return dequantize_t(q, s, static_cast<__half*>(out), M, K, block, st);
        case BI8_F32: return dequantize_t(q, s, static_cast<float*>(out), M, K, block, st);
    }
    return fail(BI8_ERR_DTYPE, "dequantize: unknown dtype code %d", dt);
}

}  // namespace bi8
