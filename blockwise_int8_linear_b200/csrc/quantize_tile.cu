// Tile quantizer: column-wise (fused transpose) quantize, and the dual quantizer that also produces the row-wise
// result from the same read of the input.
//
// Semantics (paths inside the reference project):
//   column-wise  block_linear.py:93-94, 100-103   x.t().contiguous() followed by the row-wise quantizer
//   row-wise     triton_functions.py:382-406      scale = max|x| over the block, q = rint(127 * (x / scale))
// Both results are bit-identical to the single-purpose kernels of quantize.cu (same BlockQ arithmetic).
//
// Persistent CTAs walk over tiles of 128 rows x 128 columns of a 16-bit input:
//   * one elected thread fetches the tile with two TMA loads (64 columns = 128 bytes wide each, 128-byte swizzle) that
//     complete on an mbarrier; rows and columns outside the tensor arrive as zeros;
//   * column-wise: a thread owns a pair of adjacent columns and 32 rows.  It reads them as 32 four-byte words (all lanes
//     of a warp read one row: conflict free under the swizzle), takes the absmax of both columns with packed 16-bit
//     max instructions, exchanges it with the other row groups of its block through shared memory, and quantizes
//     both columns at once with packed fp32 arithmetic.  The bytes go into a transposed tile [column][row];
//   * row-wise (dual only): a thread owns 64 consecutive columns of one row (16-byte loads, eight rows per
//     quarter-warp: conflict free under the swizzle) and writes 64 bytes into a row-major tile;
//   * the two int8 tiles leave with one TMA store each (128-byte swizzle again, so that the transposed writes do not
//     pile up on a few banks); tile parts outside the tensors are clipped by the store.
// The input tile has three stages (two in the column-wise kernel), so the next loads are in flight while a tile is quantized;
// in the dual kernel the two quantizations run side by side in two groups of 256 threads (one CTA of 512 threads per SM;
// the column-wise kernel alone runs two CTAs of 256).
#include "bi8_common.cuh"
#include "quant_math.cuh"
#include "tc_common.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

namespace bi8 {
namespace {

using namespace ptx;

constexpr int kQT = 128;          // tile edge (rows and columns)
constexpr int kQThreads = 256;
enum { QW_LOAD = 1, QW_EMPTY = 2 };

// shared memory layout (offsets from a 1024-byte aligned base) for NST input stages
constexpr uint32_t kInStage = 2 * kQT * 128;          // two sub-tiles [128 rows][128 bytes]
template <int NST>
struct QLayout {
    static constexpr uint32_t in_off = 0;
    static constexpr uint32_t outc_off = NST * kInStage;              // [128 columns][128 row bytes]
    static constexpr uint32_t ex_off = outc_off + kQT * 128;          // absmax exchange [4 row groups][128 columns] fp32
    static constexpr uint32_t bar_off = ex_off + 4 * kQT * 4;         // 2 * NST barriers and the abort flag
    static constexpr uint32_t outr_off = bar_off + 1024;              // [128 rows][128 column bytes]   (dual only)
    static constexpr uint32_t bytes_col = outr_off, bytes_dual = outr_off + kQT * 128;
    static_assert(outr_off % 1024 == 0 && outc_off % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
};

// byte offset of 16-byte chunk `chunk` of row `row` in a [rows][128 bytes] tile written or read by TMA with the 128-byte swizzle
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

template <typename T>
struct Pk;
template <>
struct Pk<__nv_bfloat16> {
    // max(|a|, m) on both 16-bit halves; a NaN operand is ignored, like fmaxf
    static __device__ __forceinline__ uint32_t absmax(uint32_t a, uint32_t m) {
        __nv_bfloat162 r = __hmax2(__habs2(*reinterpret_cast<__nv_bfloat162*>(&a)), *reinterpret_cast<__nv_bfloat162*>(&m));
        return *reinterpret_cast<uint32_t*>(&r);
    }
    static __device__ __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
        lo = bf16lo(w);
        hi = bf16hi(w);
    }
};
template <>
struct Pk<__half> {
    static __device__ __forceinline__ uint32_t absmax(uint32_t a, uint32_t m) {
        __half2 r = __hmax2(__habs2(*reinterpret_cast<__half2*>(&a)), *reinterpret_cast<__half2*>(&m));
        return *reinterpret_cast<uint32_t*>(&r);
    }
    static __device__ __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
        float2 f = __half22float2(*reinterpret_cast<__half2*>(&w));
        lo = f.x;
        hi = f.y;
    }
};

// Quantizer of a pair of values with (possibly different) block scales, on packed fp32 pairs.  The same operations, in
// the same order and each rounded on its own, as BlockQ::q: q0 = x*r, e = fma(-s, q0, x), y = fma(e, r, q0),
// z = 127*y, z + magic (written as fma(z, 1, magic) so that the multiply cannot be contracted into the addition).
struct PairQ {
    BlockQ lo, hi;
    uint64_t r2, ns2;
    bool fast;
    __device__ __forceinline__ void set(float amax_lo, float amax_hi) {
        lo.set(amax_lo, true);
        hi.set(amax_hi, true);
        fast = lo.fast && hi.fast;
        r2 = f2_pack(lo.rcp, hi.rcp);
        ns2 = f2_pack(-amax_lo, -amax_hi);
    }
    // FAST is this->fast, tested once by the caller around its whole loop rather than once per pair
    template <bool FAST>
    __device__ __forceinline__ void q(float xlo, float xhi, uint32_t& blo, uint32_t& bhi) const {
        if (FAST) {
            const uint64_t c127 = f2_pack(127.0f, 127.0f), cmagic = f2_pack(kMagic, kMagic), cone = f2_pack(1.0f, 1.0f);
            const uint64_t v2 = f2_pack(xlo, xhi);
            const uint64_t q0 = f2_mul(v2, r2);
            const uint64_t e = f2_fma(ns2, q0, v2);
            const uint64_t y = f2_fma(e, r2, q0);
            f2_bits(f2_fma(f2_mul(c127, y), cone, cmagic), blo, bhi);
        } else {
            blo = lo.q(xlo);
            bhi = hi.q(xhi);
        }
    }
};

// Barrier among the `n` threads of one role (named barrier `id`) that also tells every one of them whether all of them
// came with `ok` set: a wait that ran out in some thread ends the loop in all threads of the role, so that no thread is
// left waiting at a barrier the others will never reach.
__device__ __forceinline__ bool role_barrier_all(int id, int n, bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, %2, %3, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"(ok ? 1u : 0u), "r"(id), "r"(n)
        : "memory");
    return r != 0u;
}
__device__ __forceinline__ void role_barrier(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// Persistent CTAs walk over the tiles; the input tile has two or three stages (full / empty mbarriers per stage, the
// loads of the next tiles are in flight while the current one is quantized, and a stage is released as soon as every thread
// has its part of it in registers).  256 threads do the column-wise work; in the dual kernel 256 more do the row-wise work on the
// same tile at the same time.  Each role has its own named barrier and its own elected thread for the TMA store of its
// output tile, so neither waits for the other.
template <typename T, int B, bool DUAL>
__global__ void __launch_bounds__(DUAL ? 2 * kQThreads : kQThreads, DUAL ? 1 : 2)
quantize_tile_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmQc,
                     const __grid_constant__ CUtensorMap tmQr, float* __restrict__ s_col, float* __restrict__ s_row, int R, int C,
                     int col_tiles, int num_tiles, int* status) {
    static_assert(B == 32 || B == 64 || B == 128, "block sizes of the tile quantizer");
    constexpr int NT = DUAL ? 2 * kQThreads : kQThreads;
    constexpr int NST = DUAL ? 3 : 2;                      // input stages: the loads of the next NST - 1 tiles are in flight
    using L = QLayout<NST>;
    constexpr long long kLimit = 2000000000ll;            // about a second at the boost clock
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_dyn + (base - raw);
    const uint32_t bars = base + L::bar_off, abort_flag = bars + 16u * NST;
    auto full = [&](int s) { return bars + 8u * (uint32_t)s; };
    auto empty = [&](int s) { return bars + 8u * (uint32_t)(NST + s); };
    const int tid = threadIdx.x, lane = tid & 31;

    auto issue = [&](int t, int stage) {
        const int c0 = (t % col_tiles) * kQT, r0 = (t / col_tiles) * kQT;
        const uint32_t dst = base + L::in_off + (uint32_t)stage * kInStage;
        mbar_expect_tx(full(stage), kInStage);
        tma_load_2d(dst, &tmX, full(stage), c0, r0);
        tma_load_2d(dst + kQT * 128, &tmX, full(stage), c0 + 64, r0);
    };
    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), NT);
        }
        sts_u32(abort_flag, 0u);
        mbar_fence_init();
        fence_proxy_async_smem();
        for (int s = 0; s < NST - 1; ++s) {
            const int64_t t0 = (int64_t)blockIdx.x + (int64_t)s * gridDim.x;
            if (t0 < num_tiles) issue((int)t0, s);
        }
    }
    __syncthreads();

    const bool col_role = tid < kQThreads;
    const int rt_id = col_role ? 1 : 2;                   // the role's named barrier
    const int rtid = col_role ? tid : tid - kQThreads;    // thread index inside the role
    int fail_code = 0;
    bool ok = true;
    int it = 0, cur = 0;
    uint32_t par = 0;                                      // parity of stage `cur`'s full barrier for this use
    for (int64_t t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
        if (tid == 0) {
            // the tile NST - 1 iterations ahead goes into the stage that was read in the previous iteration
            const int64_t tn = t + (int64_t)(NST - 1) * gridDim.x;
            if (tn < num_tiles) {
                const int sn = cur == 0 ? NST - 1 : cur - 1;
                if (it >= 1) ok = mbar_wait(empty(sn), (uint32_t)(((it - 1) / NST) & 1), abort_flag, kLimit);
                if (ok) issue((int)tn, sn);
                else fail_code = QW_EMPTY;
            }
        }
        if (ok) {
            ok = mbar_wait(full(cur), par, abort_flag, kLimit);
            if (!ok) fail_code = QW_LOAD;
        }
        const int c0 = (int)(t % col_tiles) * kQT, r0 = (int)(t / col_tiles) * kQT;
        const uint32_t in_tile = base + L::in_off + (uint32_t)cur * kInStage;
        const int this_stage = cur;
        if (++cur == NST) { cur = 0; par ^= 1u; }

        if (col_role) {
            // ---------------- column-wise ----------------
            const int p = rtid & 63, g = rtid >> 6;        // column pair, group of 32 rows
            const int h = p >> 5, w = p & 31;              // sub-tile and word of the 128-byte row
            const uint32_t in = in_tile + (uint32_t)(h * kQT * 128) + (uint32_t)((w & 3) * 4);
            uint32_t v[32];
            uint32_t m2 = 0u;
            if (ok) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int r = g * 32 + i;
                    v[i] = lds_u32(in + swz(r, w >> 2));
                    m2 = Pk<T>::absmax(v[i], m2);
                }
                mbar_arrive(empty(this_stage));            // this thread's part of the stage is in registers
            }
            float alo, ahi;
            Pk<T>::unpack(m2, alo, ahi);
            float2* ex = reinterpret_cast<float2*>(base_ptr + L::ex_off);
            if (B > 32) ex[g * 64 + p] = make_float2(alo, ahi);
            // the previous tile's store must have read the output tile before it is written again
            if (rtid == 0) tma_store_wait_read();
            ok = role_barrier_all(rt_id, kQThreads, ok);
            if (!ok) break;
            if (B > 32) {
                constexpr int GPB = B / 32;                // row groups per block
                const int g0 = (g / GPB) * GPB;
#pragma unroll
                for (int k = 0; k < GPB; ++k) {
                    const float2 o = ex[(g0 + k) * 64 + p];
                    alo = fmaxf(alo, o.x);
                    ahi = fmaxf(ahi, o.y);
                }
            }
            PairQ pq;
            pq.set(alo, ahi);
            const int c = 2 * p;
            const uint32_t outc = base + L::outc_off;
            auto quantize_cols = [&](auto fast_tag) {
                constexpr bool FAST = decltype(fast_tag)::value;
#pragma unroll
                for (int part = 0; part < 2; ++part) {     // 16 rows = one 16-byte piece of each column's output row
                    uint32_t wl[4], wh[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint32_t bl[4], bh[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            float xlo, xhi;
                            Pk<T>::unpack(v[part * 16 + k * 4 + u], xlo, xhi);
                            pq.template q<FAST>(xlo, xhi, bl[u], bh[u]);
                        }
                        wl[k] = pack4(bl[0], bl[1], bl[2], bl[3]);
                        wh[k] = pack4(bh[0], bh[1], bh[2], bh[3]);
                    }
                    sts_v4(outc + swz(c, g * 2 + part), wl[0], wl[1], wl[2], wl[3]);
                    sts_v4(outc + swz(c + 1, g * 2 + part), wh[0], wh[1], wh[2], wh[3]);
                }
            };
            if (pq.fast) quantize_cols(std::true_type{});
            else quantize_cols(std::false_type{});
            // scales [ceil(R/B), C]: the first row group of each block writes the pair
            if ((g % (B / 32)) == 0) {
                const int rb = r0 + g * 32;
                if (rb < R && c0 + c < C) {
                    float* dst = s_col + (int64_t)(rb / B) * C + c0 + c;
                    if (c0 + c + 1 < C && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
                        *reinterpret_cast<float2*>(dst) = make_float2(alo, ahi);
                    } else {
                        dst[0] = alo;
                        if (c0 + c + 1 < C) dst[1] = ahi;
                    }
                }
            }
            fence_proxy_async_smem();
            role_barrier(rt_id, kQThreads);
            if (rtid == 0) {
                tma_store_2d(&tmQc, outc, r0, c0);
                tma_store_commit();
            }
        } else {
            // ---------------- row-wise ----------------
            const int rwarp = rtid >> 5;
            const int row = rwarp * 16 + (lane & 7) + 8 * (lane >> 4), half = (lane >> 3) & 1;
            const uint32_t in = in_tile + (uint32_t)(half * kQT * 128);
            uint32_t v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
            if (ok) {
#pragma unroll
                for (int k = 0; k < 8; ++k) lds_v4(in + swz(row, k), v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
                mbar_arrive(empty(this_stage));
            }
            constexpr int NBT = B == 32 ? 2 : 1;           // blocks inside the thread's 64 columns
            float amax[NBT];
#pragma unroll
            for (int b = 0; b < NBT; ++b) {
                uint32_t m2 = 0u;
#pragma unroll
                for (int i = 0; i < 32 / NBT; ++i) m2 = Pk<T>::absmax(v[b * (32 / NBT) + i], m2);
                float lo, hi;
                Pk<T>::unpack(m2, lo, hi);
                amax[b] = fmaxf(lo, hi);
            }
            if (B == 128) amax[0] = fmaxf(amax[0], __shfl_xor_sync(0xffffffffu, amax[0], 8));   // the row's other half
            if (rtid == 0) tma_store_wait_read();
            ok = role_barrier_all(rt_id, kQThreads, ok);
            if (!ok) break;
            const uint32_t outr = base + L::outr_off;
#pragma unroll
            for (int b = 0; b < NBT; ++b) {
                PairQ pq;
                pq.set(amax[b], amax[b]);
                auto quantize_row = [&](auto fast_tag) {
                    constexpr bool FAST = decltype(fast_tag)::value;
#pragma unroll
                    for (int k = 0; k < 4 / NBT; ++k) {
                        uint32_t wd[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int i = b * (32 / NBT) + k * 8 + u * 2;
                            float x0, x1, x2, x3;
                            uint32_t b0, b1, b2, b3;
                            Pk<T>::unpack(v[i], x0, x1);
                            Pk<T>::unpack(v[i + 1], x2, x3);
                            pq.template q<FAST>(x0, x1, b0, b1);
                            pq.template q<FAST>(x2, x3, b2, b3);
                            wd[u] = pack4(b0, b1, b2, b3);
                        }
                        sts_v4(outr + swz(row, half * 4 + b * (4 / NBT) + k), wd[0], wd[1], wd[2], wd[3]);
                    }
                };
                if (pq.fast) quantize_row(std::true_type{});
                else quantize_row(std::false_type{});
            }
            // scales [ceil(C/B), R] (transposed): eight consecutive rows per quarter-warp
            if (r0 + row < R) {
#pragma unroll
                for (int b = 0; b < NBT; ++b) {
                    const int col = c0 + half * 64 + b * 32;
                    if (col < C && !(B == 128 && half == 1)) s_row[(int64_t)(col / B) * R + r0 + row] = amax[b];
                }
            }
            fence_proxy_async_smem();
            role_barrier(rt_id, kQThreads);
            if (rtid == 0) {
                tma_store_2d(&tmQr, outr, c0, r0);
                tma_store_commit();
            }
        }
    }
    // shared memory must stay valid until the last stores have read it
    if (rtid == 0) tma_store_wait_read();
    if (!ok && rtid == 0 && fail_code != 0) report_timeout(status, abort_flag, fail_code);
}

// int8 [rows, cols] row-major, contiguous rows (cols a multiple of 16, 16-byte aligned base) -> boxes of 128 x 128 bytes, 128-byte swizzle
int make_q_map(CUtensorMap* map, int8_t* ptr, int64_t rows, int64_t cols) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    ensure_current_context();
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)cols};
    cuuint32_t box[2] = {128, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, ptr, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled (int8 tile) failed with CUresult %d", (int)r);
    return BI8_OK;
}

// 16-bit [rows, cols] row-major with row pitch ld elements -> boxes of 64 columns x 128 rows, 128-byte swizzle
int make_x_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    ensure_current_context();
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BI8_ERR_CUDA, "cuTensorMapEncodeTiled (input tile) failed with CUresult %d", (int)r);
    return BI8_OK;
}

// Encoded maps are looked up in the library's map table first (kinds 5 and 6 there): a training step quantizes tensors of
// the same few shapes at addresses the allocator keeps handing back, and an encode is a driver call of a few microseconds.
int cached_x_map(CUtensorMap* map, int dev, const void* ptr, int64_t rows, int64_t cols, int64_t ld) {
    const MapKey key{dev, 5, ptr, rows, cols, ld, 128, 64};
    if (map_cache().find(key, map)) return BI8_OK;
    const int rc = make_x_map(map, ptr, rows, cols, ld);
    if (rc == BI8_OK) map_cache().put(key, *map);
    return rc;
}
int cached_q_map(CUtensorMap* map, int dev, int8_t* ptr, int64_t rows, int64_t cols) {
    const MapKey key{dev, 6, ptr, rows, cols, cols, 128, 128};
    if (map_cache().find(key, map)) return BI8_OK;
    const int rc = make_q_map(map, ptr, rows, cols);
    if (rc == BI8_OK) map_cache().put(key, *map);
    return rc;
}

template <typename T, int B, bool DUAL>
int launch_tile(const CUtensorMap& tx, const CUtensorMap& tqc, const CUtensorMap& tqr, float* s_col, float* s_row, int64_t R,
                int64_t C, cudaStream_t st) {
    const int64_t ctiles = (C + kQT - 1) / kQT, rtiles = (R + kQT - 1) / kQT;
    if (ctiles * rtiles >= (1ll << 31)) return fail(BI8_ERR_SHAPE, "quantize: grid too large");
    constexpr size_t smem = (DUAL ? QLayout<3>::bytes_dual : QLayout<2>::bytes_col) + 1024;
    static SmemOptIn opt_in;
    const int rc = opt_in.ensure(quantize_tile_kernel<T, B, DUAL>, smem);
    if (rc != BI8_OK) return rc;
    int* status = device_status_ptr();
    if (!status) return BI8_ERR_CUDA;
    const DeviceInfo di = device_info();
    const int64_t tiles = ctiles * rtiles;
    const int64_t resident = (int64_t)(DUAL ? 1 : 2) * di.sms;                 // CTAs that fit at once
    const int grid = (int)(tiles < resident ? tiles : resident);
    quantize_tile_kernel<T, B, DUAL><<<grid, DUAL ? 2 * kQThreads : kQThreads, smem, st>>>(tx, tqc, tqr, s_col, s_row, (int)R, (int)C,
                                                                                        (int)ctiles, (int)tiles, status);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

template <typename T>
int tile_dispatch(const void* x, int64_t ldx, int8_t* q_col, float* s_col, int8_t* q_row, float* s_row, int64_t R, int64_t C, int block,
                  cudaStream_t st) {
    CUtensorMap tx, tqc, tqr;
    int dev = 0;
    BI8_CUDA_TRY(cudaGetDevice(&dev));
    int rc = cached_x_map(&tx, dev, x, R, C, ldx);
    if (rc != BI8_OK) return rc;
    rc = cached_q_map(&tqc, dev, q_col, C, R);
    if (rc != BI8_OK) return rc;
    tqr = tqc;
    const bool dual = q_row != nullptr;
    if (dual) {
        rc = cached_q_map(&tqr, dev, q_row, R, C);
        if (rc != BI8_OK) return rc;
    }
#define BI8_TILE(BB)                                                                                  \
    if (block == BB)                                                                                  \
        return dual ? launch_tile<T, BB, true>(tx, tqc, tqr, s_col, s_row, R, C, st)                  \
                    : launch_tile<T, BB, false>(tx, tqc, tqr, s_col, s_row, R, C, st);
    BI8_TILE(32) BI8_TILE(64) BI8_TILE(128)
#undef BI8_TILE
    return fail(BI8_ERR_BLOCK, "tile quantizer supports block 32, 64, 128 (got %d)", block);
}

}  // namespace

// The tile quantizer needs what its tensor maps need: a 16-bit input with 16-byte aligned base and row pitch, and int8
// outputs whose rows (R bytes for the transposed one, C bytes for the row-wise one) are multiples of 16 bytes.
bool quantize_tile_applicable(const void* x, int dt, int64_t ldx, const void* q_col, const void* q_row, int64_t R, int64_t C, int block) {
    if (dt != BI8_BF16 && dt != BI8_F16) return false;
    if (block != 32 && block != 64 && block != 128) return false;
    if (R <= 0 || C <= 0 || R >= (1ll << 31) || C >= (1ll << 31)) return false;
    if (!aligned(x, 16) || (ldx * 2) % 16 != 0 || !aligned(q_col, 16) || R % 16 != 0) return false;
    if (q_row != nullptr && (!aligned(q_row, 16) || C % 16 != 0)) return false;
    return device_info().ok;
}

int launch_quantize_tile(const void* x, int dt, int64_t ldx, int8_t* q_col, float* s_col, int8_t* q_row, float* s_row, int64_t R,
                         int64_t C, int block, cudaStream_t st) {
    if (dt == BI8_BF16) return tile_dispatch<__nv_bfloat16>(x, ldx, q_col, s_col, q_row, s_row, R, C, block, st);
    if (dt == BI8_F16) return tile_dispatch<__half>(x, ldx, q_col, s_col, q_row, s_row, R, C, block, st);
    return fail(BI8_ERR_DTYPE, "tile quantizer takes bf16 or fp16 input");
}

}  // namespace bi8
