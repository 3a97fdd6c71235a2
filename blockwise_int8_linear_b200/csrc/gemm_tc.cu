// Int8 block GEMM with fused dequantize on the sm_100a tensor cores.
//
// Replaces the reference kernel at triton_functions.py:69-139 (path inside the reference project):
//   P_j = A[:, jB:(j+1)B] . Bt[:, jB:(j+1)B]^T      exact int32 (line 115)
//   acc += sB[j,n] * sA[j,m] * float(P_j) / 127^2   fp32, j ascending (line 120)
//   C = cast(acc) (+ cast(bias))                    (lines 125-131)
//
// One persistent CTA per SM works on 128 x 160 output tiles.  Warp roles:
//   warp 0      TMA producer: 128-byte-swizzled K-major tiles of A (128 rows) and Bt (160 rows), 128 K-bytes
//               per stage, ring of kStages stages
//   warp 1      issues tcgen05.mma kind::i8 (M128 N160 K32): the MMAs of one quantisation block accumulate
//               into one of three s32 accumulators in tensor memory (the hand-off latency of a block is
//               several times its MMA time, so more than two blocks have to be in flight), then a commit hands that
//               accumulator to the promotion warps
//   warps 2-3   stage the block scales of the tile (sA: 128 rows, sB: 160 columns per block) in shared memory
//   warps 4-19  promotion + epilogue: read an accumulator from tensor memory (each warp owns 32 rows x 40
//               columns), fold it into fp32 accumulators held in registers, release the accumulator; after
//               the last block convert, add bias and store
// Registers are moved from warps 0-3 to warps 4-19 with setmaxnreg (40 fp32 accumulators per thread); four
// promotion warps per scheduler cover each other's tensor-memory load latency.
//
// Seeded conversion (default): the promotion warps refill a drained accumulator with the bit pattern of
// 1.5*2^23 and every MMA accumulates on top of it.  Integer addition on that pattern is exact float
// arithmetic while |P| < 2^22, so the word read back is the float 1.5*2^23 + P and
//   t = fma(word, s, -1.5*2^23 * s) = fl(P * s)
// needs no int->float conversion.  s = sA[j,m]/127^2 rounded to 22 significant bits makes 1.5*2^23*s exact.
#include "bi8_common.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <cstring>

namespace bi8 {
namespace {

using namespace ptx;

constexpr int kBM = 128;                 // tile rows
constexpr int kBN = 160;                 // tile columns (40 per promotion warp: accumulators fit the register budget)
constexpr int kAccBufs = 3;              // s32 accumulators in tensor memory (3 x 160 of the 512 columns)
constexpr int kAccStride = kBN;          // tensor-memory columns between consecutive accumulators
constexpr int kProbeN = 256;             // N of the issue-rate probe's MMAs
constexpr int kStages = 5;
constexpr int kScaleStages = 4;
constexpr int kEpiWarps = 16;             // 4 lane quarters x 4 column slices of 64
constexpr int kThreadsTc = (4 + kEpiWarps) * 32;
constexpr int kEpiCols = kBN / (kEpiWarps / 4);   // columns owned by one promotion warp
constexpr uint32_t kABytes = kBM * kBK;  // 16 KiB
constexpr uint32_t kBBytes = kBN * kBK;  // 20 KiB
constexpr uint32_t kSeedBits = 0x4B400000u;   // float 1.5 * 2^23
constexpr float kSeedF = 12582912.0f;

struct TcParams {
    const float* sA;
    const float* sB;
    const void* bias;
    void* C;
    int32_t* partials;
    int* status;
    int64_t ldc;
    int M, N, K, nb;
    int tiles_m, tiles_n;
    int out_dtype, bias_dtype;
    int vec_store;      // C base and row pitch allow 16-byte stores
    int vec_scales;     // sA, sB and their row lengths allow 16-byte loads
    int ksplit;         // > 1: the K stages are divided over ksplit work items per tile (split-K)
    int stages_per_split;
    float* ws;          // split-K: fp32 partial results [ksplit, M, N]
};

struct Smem {
    // byte offsets from the 1024-aligned base of dynamic shared memory
    __host__ __device__ static constexpr uint32_t a_off(int s) { return (uint32_t)s * (kABytes + kBBytes); }
    __host__ __device__ static constexpr uint32_t b_off(int s) { return a_off(s) + kABytes; }
    static constexpr uint32_t scale_off = kStages * (kABytes + kBBytes);
};

template <int QB>
struct Geo {
    static constexpr int BPS = kBK / QB;                        // quantisation blocks per stage
    static constexpr int MMAS = QB / 32;                        // MMAs (K = 32) per block
    static constexpr int SC_FLOATS = BPS * (kBM + kBN);         // scale floats per stage
    static constexpr uint32_t bar_off = Smem::scale_off + kScaleStages * SC_FLOATS * 4;
    // barrier slots (8 bytes each)
    static constexpr int FULL_AB = 0, EMPTY_AB = kStages, ACC_FULL = 2 * kStages, ACC_EMPTY = 2 * kStages + kAccBufs,
                         SC_FULL = 2 * kStages + 2 * kAccBufs, SC_EMPTY = 2 * kStages + 2 * kAccBufs + kScaleStages,
                         NBARS = 2 * kStages + 2 * kAccBufs + 2 * kScaleStages;
    static constexpr uint32_t misc_off = bar_off + NBARS * 8;   // tmem holder (4 B) + abort flag (4 B)
    static constexpr uint32_t total = misc_off + 16;
};

// Work item -> tile and K-stage range.  Items of one split are consecutive, so CTAs that run together work on
// different tiles of the same K range.
__device__ __forceinline__ void item_range(int item, int num_tiles, int nks, int stages_per_split, int& tile, int& split,
                                           int& ks0, int& ks1) {
    tile = item % num_tiles;
    split = item / num_tiles;
    ks0 = split * stages_per_split;
    ks1 = ks0 + stages_per_split;
    if (ks1 > nks) ks1 = nks;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int& m0, int& n0) {
    // consecutive tiles (CTAs that run together) share a column panel of Bt and sweep the rows of A
    m0 = (tile % tiles_m) * kBM;
    n0 = (tile / tiles_m) * kBN;
}

template <int QB, int MODE, bool SEED>
__global__ void __launch_bounds__(kThreadsTc, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcParams p) {
    using G = Geo<QB>;
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    // dynamic shared memory is only guaranteed 16-byte aligned: round up to the swizzle atom
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_dyn + (base - raw);
    float* sc_ring = reinterpret_cast<float*>(base_ptr + Smem::scale_off);
    const uint32_t sc_ring_u32 = base + Smem::scale_off;
    const uint32_t bars = base + G::bar_off;
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(base_ptr + G::misc_off);
    const uint32_t abort_flag = base + G::misc_off + 4;
    auto bar = [&](int slot) -> uint32_t { return bars + 8u * (uint32_t)slot; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int nks = (p.K + kBK - 1) / kBK;
    const int num_items = num_tiles * p.ksplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(G::FULL_AB + s), 1);
            mbar_init(bar(G::EMPTY_AB + s), 1);
        }
        for (int b = 0; b < kAccBufs; ++b) {
            mbar_init(bar(G::ACC_FULL + b), 1);
            mbar_init(bar(G::ACC_EMPTY + b), kEpiWarps);
        }
        for (int s = 0; s < kScaleStages; ++s) {
            mbar_init(bar(G::SC_FULL + s), 64);      // every lane of the two scale warps
            mbar_init(bar(G::SC_EMPTY + s), kEpiWarps);
        }
        sts_u32(abort_flag, 0u);
        sts_u32(base + G::misc_off + 8, 0u);       // a flag nobody raises, for waits that must not be cut short
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 2) {
        tmem_alloc(smem_u32((const void*)tmem_holder), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    // setmaxnreg moves registers inside the CTA's launch-time allocation (kThreadsTc * 96): the totals after
    // the moves must not exceed it, or setmaxnreg.inc blocks forever.
    static_assert(128 * 24 + (kThreadsTc - 128) * 112 <= kThreadsTc * 96, "register budget exceeds the launch allocation");
    if (warp < 4) {
        setmaxnreg_dec<24>();
        // Whole warps run the producer and MMA loops convergently and one lane issues: lanes parked at the final
        // barrier while a sibling lane loops make that loop crawl.
        if (warp == 0) {
            // ---------------- TMA producer ----------------
            int stage = 0;
            uint32_t phase = 0;
            int last_parity[kStages];
#pragma unroll
            for (int s = 0; s < kStages; ++s) last_parity[s] = -1;
            bool ok = true;
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                int tile, split, ks0, ks1, m0, n0;
                item_range(item, num_tiles, nks, p.stages_per_split, tile, split, ks0, ks1);
                tile_coords(tile, p.tiles_m, m0, n0);
                for (int ks = ks0; ks < ks1; ++ks) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(G::EMPTY_AB + stage), phase ^ 1u, abort_flag));
                    if (!ok) {
                        if (lane == 0) report_timeout(p.status, abort_flag, W_EMPTY_AB);
                        break;
                    }
                    if (lane == 0) {
                        mbar_expect_tx(bar(G::FULL_AB + stage), kABytes + kBBytes);
                        tma_load_2d(base + Smem::a_off(stage), &tmA, bar(G::FULL_AB + stage), ks * kBK, m0);
                        tma_load_2d(base + Smem::b_off(stage), &tmB, bar(G::FULL_AB + stage), ks * kBK, n0);
                    }
                    __syncwarp();
#pragma unroll
                    for (int s = 0; s < kStages; ++s)
                        if (s == stage) last_parity[s] = (int)phase;
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // do not leave while our own copies may still land in this CTA's shared memory
#pragma unroll
                for (int s = 0; s < kStages; ++s) {
                    if (last_parity[s] >= 0) {
                        (void)mbar_wait(bar(G::FULL_AB + s), (uint32_t)last_parity[s], base + G::misc_off + 8, 200000000ll);
                    }
                }
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            constexpr uint32_t idesc = umma_idesc_i8(kBM, kBN);
            int stage = 0, accbuf = 0;
            uint32_t phase = 0, accphase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                int tile, split, ks0, ks1;
                item_range(item, num_tiles, nks, p.stages_per_split, tile, split, ks0, ks1);
                for (int ks = ks0; ks < ks1 && ok; ++ks) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(G::FULL_AB + stage), phase, abort_flag));
                    if (!ok) {
                        if (lane == 0) report_timeout(p.status, abort_flag, W_FULL_AB);
                        break;
                    }
                    tc_fence_after();
                    const uint64_t adesc = umma_desc_k_sw128(base + Smem::a_off(stage));
                    const uint64_t bdesc = umma_desc_k_sw128(base + Smem::b_off(stage));
#pragma unroll
                    for (int blk = 0; blk < G::BPS; ++blk) {
                        if (ks * G::BPS + blk >= p.nb) break;
                        ok = __all_sync(0xffffffffu, mbar_wait(bar(G::ACC_EMPTY + accbuf), accphase, abort_flag));
                        if (!ok) {
                            if (lane == 0) report_timeout(p.status, abort_flag, W_ACC_EMPTY);
                            break;
                        }
                        tc_fence_after();
                        if (lane == 0) {
#pragma unroll
                            for (int i = 0; i < G::MMAS; ++i) {
                                const uint64_t koff = (uint64_t)((blk * G::MMAS + i) * 32 / 16);
                                mma_i8(tmem_base + (uint32_t)accbuf * kAccStride, adesc + koff, bdesc + koff, idesc,
                                       (SEED || i > 0) ? 1u : 0u);
                            }
                            tc_commit(bar(G::ACC_FULL + accbuf));
                        }
                        __syncwarp();
                        if (++accbuf == kAccBufs) { accbuf = 0; accphase ^= 1u; }
                    }
                    if (!ok) break;
                    if (lane == 0) tc_commit(bar(G::EMPTY_AB + stage));
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        } else {
            // ---------------- scale loaders: warp 2 stages sA (128 rows per block), warp 3 sB (160 columns) ----------
            const bool is_a = (warp == 2);
            const float* src = is_a ? p.sA : p.sB;
            const int extent = is_a ? p.M : p.N;          // row length of the scale tensor
            const int width = is_a ? kBM : kBN;           // floats per block taken by this warp
            const int dst_off = is_a ? 0 : kBM;
            int sstage = 0;
            uint32_t sphase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                int tile, split, ks0, ks1, m0, n0;
                item_range(item, num_tiles, nks, p.stages_per_split, tile, split, ks0, ks1);
                tile_coords(tile, p.tiles_m, m0, n0);
                const int x0 = is_a ? m0 : n0;
                for (int ks = ks0; ks < ks1; ++ks) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(G::SC_EMPTY + sstage), sphase ^ 1u, abort_flag));
                    if (!ok) {
                        if (lane == 0) report_timeout(p.status, abort_flag, W_SC_EMPTY);
                        break;
                    }
                    // asynchronous copies: the warp does not wait for the data, so the loads of several stages are
                    // in flight at once; each lane's arrival on the stage's barrier fires when its copies have landed
                    const uint32_t dst = sc_ring_u32 + (uint32_t)((sstage * G::SC_FLOATS + dst_off) * 4);
                    if (src == nullptr) {
                        // partial-sum dump: no scales, the ring content is never used
                    } else if (p.vec_scales) {
                        const int nv = G::BPS * width / 4;                   // 16-byte pieces in this warp's part
                        for (int idx = lane; idx < nv; idx += 32) {
                            const int blk = idx / (width / 4), c4 = (idx % (width / 4)) * 4;
                            const int j = ks * G::BPS + blk;
                            const bool live = j < p.nb && x0 + c4 < extent;
                            const float* g = live ? src + (int64_t)j * extent + x0 + c4 : src;
                            cp_async_16(dst + (uint32_t)((blk * (kBM + kBN) + c4) * 4), g, live ? 16u : 0u);
                        }
                    } else {
                        for (int idx = lane; idx < G::BPS * width; idx += 32) {
                            const int blk = idx / width, c = idx % width;
                            const int j = ks * G::BPS + blk;
                            const bool live = j < p.nb && x0 + c < extent;
                            const float* g = live ? src + (int64_t)j * extent + x0 + c : src;
                            cp_async_4(dst + (uint32_t)((blk * (kBM + kBN) + c) * 4), g, live ? 4u : 0u);
                        }
                    }
                    cp_async_arrive(bar(G::SC_FULL + sstage));
                    if (++sstage == kScaleStages) { sstage = 0; sphase ^= 1u; }
                }
            }
        }
    } else {
        // ---------------- promotion + epilogue (warps 4..19) ----------------
        setmaxnreg_inc<112>();
        const int quarter = warp & 3;            // tensor-memory lanes 32*quarter .. +31 belong to this warp
        const int slice = (warp - 4) >> 2;       // columns kEpiCols*slice .. of the tile
        const int row = quarter * 32 + lane;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(slice * kEpiCols);
        const float div = 1.0f / (127.0f * 127.0f);
        uint32_t seedv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) seedv[i] = opaque_u32(kSeedBits);

        if (SEED) {
#pragma unroll
            for (int b = 0; b < kAccBufs; ++b)
#pragma unroll
                for (int c = 0; c < kEpiCols / 8; ++c) tmem_st8(t_lane + (uint32_t)(b * kAccStride + c * 8), seedv);
            tmem_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < kAccBufs; ++b) mbar_arrive(bar(G::ACC_EMPTY + b));
        }

        int accbuf = 0, sstage = 0;
        uint32_t accphase = 0, sphase = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            int tile, split, ks0, ks1, m0, n0;
            item_range(item, num_tiles, nks, p.stages_per_split, tile, split, ks0, ks1);
            tile_coords(tile, p.tiles_m, m0, n0);
            const int m = m0 + row;
            const bool warp_live = (m0 + quarter * 32) < p.M;      // small M: most warps own no valid row
            const int nbase = n0 + slice * kEpiCols;
            // kEpiCols fp32 accumulators per thread, kept as packed pairs for fma.rn.f32x2
            uint64_t acc2[kEpiCols / 2];
#pragma unroll
            for (int i = 0; i < kEpiCols / 2; ++i) acc2[i] = 0ull;

            for (int ks = ks0; ks < ks1 && ok; ++ks) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(G::SC_FULL + sstage), sphase, abort_flag));
                if (!ok) {
                    if (lane == 0) report_timeout(p.status, abort_flag, W_SC_FULL);
                    break;
                }
                const float* sc = sc_ring + sstage * G::SC_FLOATS;
                const uint32_t sc_u32 = sc_ring_u32 + (uint32_t)(sstage * G::SC_FLOATS * 4);
#pragma unroll 1
                for (int blk = 0; blk < G::BPS; ++blk) {
                    const int j = ks * G::BPS + blk;
                    if (j >= p.nb) break;
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(G::ACC_FULL + accbuf), accphase, abort_flag));
                    if (!ok) {
                        if (lane == 0) report_timeout(p.status, abort_flag, W_ACC_FULL);
                        break;
                    }
                    tc_fence_after();
                    const uint32_t t_acc = t_lane + (uint32_t)(accbuf * kAccStride);
                    if (!warp_live) {
                        // all 32 rows of this warp lie beyond M: nothing to fold, and what the MMAs leave in these
                        // tensor-memory lanes is never read
                    } else if (MODE == 1) {
#pragma unroll
                        for (int c = 0; c < kEpiCols / 8; ++c) {
                            uint32_t pv[8];
                            tmem_ld8(t_acc + (uint32_t)(c * 8), pv);
                            tmem_wait_ld();
                            if (SEED) tmem_st8(t_acc + (uint32_t)(c * 8), seedv);
                            if (m < p.M) {
                                int32_t* dst = p.partials + ((int64_t)j * p.M + m) * p.N + nbase + c * 8;
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    if (nbase + c * 8 + i < p.N)
                                        dst[i] = SEED ? (int32_t)(pv[i] - kSeedBits) : (int32_t)pv[i];
                            }
                        }
                        if (SEED) tmem_wait_st();
                    } else {
                        float sxd = __fmul_rn(lds_f32(sc_u32 + (uint32_t)((blk * (kBM + kBN) + row) * 4)), div);
                        float negc = 0.0f;
                        if (SEED) {
                            sxd = __uint_as_float((__float_as_uint(sxd) + 2u) & 0xFFFFFFFCu);   // 22 significant bits
                            negc = -__fmul_rn(kSeedF, sxd);                                      // exact
                        }
                        const uint64_t sxd2 = pack_f32x2(sxd, sxd), negc2 = pack_f32x2(negc, negc);
                        const uint32_t sw_u32 = sc_u32 + (uint32_t)((blk * (kBM + kBN) + kBM + slice * kEpiCols) * 4);
                        // 8 columns per step: one load, one re-seed store (8 resident seed registers), two 16-byte scale
                        // loads, eight packed FMAs; the next load is issued before the current chunk is folded.
                        uint32_t pa[8], pb[8];
                        tmem_ld8(t_acc, pa);
#pragma unroll
                        for (int c = 0; c < kEpiCols / 8; ++c) {
                            uint32_t(&cur)[8] = (c & 1) ? pb : pa;
                            uint32_t(&nxt)[8] = (c & 1) ? pa : pb;
                            tmem_wait_ld();
                            if (c + 1 < kEpiCols / 8) tmem_ld8(t_acc + (uint32_t)((c + 1) * 8), nxt);
                            if (SEED) tmem_st8(t_acc + (uint32_t)(c * 8), seedv);
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                uint64_t w0, w1;
                                lds_2xb64(sw_u32 + (uint32_t)((c * 2 + q) * 16), w0, w1);
                                uint64_t t0, t1;
                                if (SEED) {
                                    t0 = fma_f32x2(pack_u32x2(cur[4 * q], cur[4 * q + 1]), sxd2, negc2);
                                    t1 = fma_f32x2(pack_u32x2(cur[4 * q + 2], cur[4 * q + 3]), sxd2, negc2);
                                } else {
                                    t0 = fma_f32x2(pack_f32x2((float)(int32_t)cur[4 * q], (float)(int32_t)cur[4 * q + 1]), sxd2, 0ull);
                                    t1 = fma_f32x2(pack_f32x2((float)(int32_t)cur[4 * q + 2], (float)(int32_t)cur[4 * q + 3]), sxd2, 0ull);
                                }
                                acc2[c * 4 + q * 2] = fma_f32x2(w0, t0, acc2[c * 4 + q * 2]);
                                acc2[c * 4 + q * 2 + 1] = fma_f32x2(w1, t1, acc2[c * 4 + q * 2 + 1]);
                            }
                        }
                        if (SEED) tmem_wait_st();
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(G::ACC_EMPTY + accbuf));
                    if (++accbuf == kAccBufs) { accbuf = 0; accphase ^= 1u; }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(G::SC_EMPTY + sstage));
                if (++sstage == kScaleStages) { sstage = 0; sphase ^= 1u; }
            }
            if (!ok) break;

            if (MODE == 0 && m < p.M) {
                float acc[kEpiCols];
#pragma unroll
                for (int i = 0; i < kEpiCols / 2; ++i) unpack_f32x2(acc2[i], acc[2 * i], acc[2 * i + 1]);
                if (p.ksplit > 1) {
                    // split-K: raw fp32 partial result of this K range; cast and bias happen in the reduction
                    float* wrow = p.ws + ((int64_t)split * p.M + m) * p.N;
#pragma unroll
                    for (int g = 0; g < kEpiCols / 4; ++g) {
                        const int n = nbase + g * 4;
                        if ((p.N & 3) == 0 && n + 4 <= p.N) {
                            *reinterpret_cast<float4*>(wrow + n) = make_float4(acc[g * 4], acc[g * 4 + 1], acc[g * 4 + 2], acc[g * 4 + 3]);
                        } else {
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                                if (n + u < p.N) wrow[n + u] = acc[g * 4 + u];
                        }
                    }
                    continue;
                }
                const bool has_bias = p.bias != nullptr;
                auto bias_at = [&](int n) -> float {
                    if (p.bias_dtype == BI8_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
                    if (p.bias_dtype == BI8_F16) return __half2float(static_cast<const __half*>(p.bias)[n]);
                    return static_cast<const float*>(p.bias)[n];
                };
                if (p.out_dtype == BI8_F32) {
                    float* crow = static_cast<float*>(p.C) + (int64_t)m * p.ldc;
#pragma unroll
                    for (int g = 0; g < kEpiCols / 4; ++g) {
                        const int n = nbase + g * 4;
                        float v[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            v[u] = acc[g * 4 + u];
                            if (has_bias && n + u < p.N) v[u] = __fadd_rn(v[u], bias_at(n + u));
                        }
                        if (p.vec_store && n + 4 <= p.N) {
                            *reinterpret_cast<float4*>(crow + n) = make_float4(v[0], v[1], v[2], v[3]);
                        } else {
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                                if (n + u < p.N) crow[n + u] = v[u];
                        }
                    }
                } else {
                    const bool bf = p.out_dtype == BI8_BF16;
                    uint16_t* crow = static_cast<uint16_t*>(p.C) + (int64_t)m * p.ldc;
#pragma unroll
                    for (int g = 0; g < kEpiCols / 8; ++g) {
                        const int n = nbase + g * 8;
                        uint32_t w[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            float lo = acc[g * 8 + 2 * u], hi = acc[g * 8 + 2 * u + 1];
                            uint32_t pk = bf ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
                            if (has_bias) {
                                // the reference adds the bias after the cast, in the output type (lines 127-131)
                                float blo = (n + 2 * u < p.N) ? bias_at(n + 2 * u) : 0.0f;
                                float bhi = (n + 2 * u + 1 < p.N) ? bias_at(n + 2 * u + 1) : 0.0f;
                                if (bf) {
                                    uint32_t bb = pack_bf16x2(blo, bhi);
                                    pk = pack_bf16x2(__fadd_rn(bf16lo(pk), bf16lo(bb)), __fadd_rn(bf16hi(pk), bf16hi(bb)));
                                } else {
                                    __half2 a2 = *reinterpret_cast<__half2*>(&pk);
                                    __half2 b2 = __floats2half2_rn(blo, bhi);
                                    float2 af = __half22float2(a2), bfv = __half22float2(b2);
                                    pk = pack_f16x2(__fadd_rn(af.x, bfv.x), __fadd_rn(af.y, bfv.y));
                                }
                            }
                            w[u] = pk;
                        }
                        if (p.vec_store && n + 8 <= p.N) {
                            *reinterpret_cast<uint4*>(crow + n) = make_uint4(w[0], w[1], w[2], w[3]);
                        } else {
#pragma unroll
                            for (int u = 0; u < 8; ++u)
                                if (n + u < p.N) crow[n + u] = (uint16_t)((w[u / 2] >> (16 * (u % 2))) & 0xffffu);
                        }
                    }
                }
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Split-K reduction: C[m,n] = cast(sum_s ws[s,m,n]) (+ cast(bias[n]) in the output type).  The splits are added in
// ascending order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ ws, int ksplit, const void* __restrict__ bias,
                                                            int bias_dtype, void* __restrict__ C, int64_t ldc, int out_dtype,
                                                            int M, int N) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (int64_t)M * N) return;
    const int m = (int)(i / N), n = (int)(i % N);
    float acc = 0.0f;
    for (int s = 0; s < ksplit; ++s) acc = __fadd_rn(acc, ws[((int64_t)s * M + m) * N + n]);
    float bv = 0.0f;
    const bool hb = bias != nullptr;
    if (hb) {
        if (bias_dtype == BI8_BF16) bv = __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
        else if (bias_dtype == BI8_F16) bv = __half2float(static_cast<const __half*>(bias)[n]);
        else bv = static_cast<const float*>(bias)[n];
    }
    if (out_dtype == BI8_F32) {
        static_cast<float*>(C)[(int64_t)m * ldc + n] = hb ? __fadd_rn(acc, bv) : acc;
    } else if (out_dtype == BI8_BF16) {
        __nv_bfloat16 c = __float2bfloat16_rn(acc);
        if (hb) c = __float2bfloat16_rn(__fadd_rn(__bfloat162float(c), __bfloat162float(__float2bfloat16_rn(bv))));
        static_cast<__nv_bfloat16*>(C)[(int64_t)m * ldc + n] = c;
    } else {
        __half c = __float2half_rn(acc);
        if (hb) c = __float2half_rn(__fadd_rn(__half2float(c), __half2float(__float2half_rn(bv))));
        static_cast<__half*>(C)[(int64_t)m * ldc + n] = c;
    }
}

// Issue-rate probe: back-to-back M128 N256 K32 int8 MMAs on zeroed shared memory, no loads, no epilogue.
__global__ void __launch_bounds__(128, 1) mma_peak_probe_kernel(int iters, int* status) {
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_dyn + (base - raw);
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t holder;
    __shared__ uint32_t abort_word;
    for (uint32_t i = threadIdx.x; i < (kABytes + kProbeN * kBK) / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(base_ptr)[i] = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done_bar), 1);
        abort_word = 0;
        mbar_fence_init();
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        tmem_alloc(smem_u32(&holder), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t*)&holder;
    if (threadIdx.x == 32) {
        constexpr uint32_t idesc = umma_idesc_i8(kBM, kProbeN);
        const uint64_t adesc = umma_desc_k_sw128(base), bdesc = umma_desc_k_sw128(base + kABytes);
        for (int i = 0; i < iters; ++i) {
            const uint64_t koff = (uint64_t)((i & 3) * 2);
            mma_i8(tmem_base + (uint32_t)((i >> 2) & 1) * kProbeN, adesc + koff, bdesc + koff, idesc, (i >= 8) ? 1u : 0u);
        }
        tc_commit(smem_u32(&done_bar));
        if (!mbar_wait(smem_u32(&done_bar), 0u, smem_u32(&abort_word), 10000000000ll)) report_timeout(status, smem_u32(&abort_word), W_PROBE);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int QB, int MODE, bool SEED>
int launch_one(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int grid, cudaStream_t st) {
    constexpr size_t smem = Geo<QB>::total + 1024;
    BI8_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<QB, MODE, SEED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gemm_tc_kernel<QB, MODE, SEED><<<grid, kThreadsTc, smem, st>>>(ma, mb, p);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

template <int QB>
int launch_qb(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int grid, bool partials, bool seed,
              cudaStream_t st) {
    if (partials) return seed ? launch_one<QB, 1, true>(ma, mb, p, grid, st) : launch_one<QB, 1, false>(ma, mb, p, grid, st);
    return seed ? launch_one<QB, 0, true>(ma, mb, p, grid, st) : launch_one<QB, 0, false>(ma, mb, p, grid, st);
}

}  // namespace

// Split-K plan: when the output has fewer tiles than the device has SMs (small M), the K stages of every tile are
// divided over `ksplit` work items so that all SMs stream weights; partial results go to an fp32 workspace
// [ksplit, M, N] and a second kernel adds them in a fixed order.
namespace {
struct SplitPlan {
    int ksplit = 1;
    int stages_per_split = 0;
    size_t bytes = 0;
};
SplitPlan plan_split(int64_t M, int64_t N, int64_t K, int sms) {
    SplitPlan pl;
    const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
    const int nks = (int)((K + kBK - 1) / kBK);
    pl.stages_per_split = nks;
    if (tiles <= 0 || nks <= 1 || tiles * 2 > sms) return pl;
    int s = (int)(sms / tiles);
    if (s > nks) s = nks;
    if (s > 32) s = 32;
    while (s > 1 && (size_t)s * (size_t)M * (size_t)N * 4 > (size_t)256 << 20) --s;
    if (s <= 1) return pl;
    const int spp = (nks + s - 1) / s;
    pl.ksplit = (nks + spp - 1) / spp;
    pl.stages_per_split = spp;
    pl.bytes = pl.ksplit > 1 ? (size_t)pl.ksplit * (size_t)M * (size_t)N * 4 : 0;
    return pl;
}
}  // namespace

size_t gemm_tc_workspace_bytes(const GemmArgs& g) {
    const DeviceInfo di = device_info();
    if (!di.ok || g.partials != nullptr) return 0;
    return plan_split(g.M, g.N, g.K, di.sms).bytes;
}

bool gemm_tc_applicable(const GemmArgs& g, const char** why) {
    auto no = [&](const char* w) {
        if (why) *why = w;
        return false;
    };
    if (g.block != 32 && g.block != 64 && g.block != 128) return no("block size is not 32, 64 or 128");
    if (g.M >= (1ll << 31) - 256 || g.N >= (1ll << 31) - 256 || g.K >= (1ll << 31) - 256) return no("a dimension exceeds 2^31");
    if (!aligned(g.A, 16) || !aligned(g.Bt, 16)) return no("operand base address is not 16-byte aligned");
    if (g.lda % 16 != 0 || g.ldb % 16 != 0) return no("operand row pitch is not a multiple of 16 bytes");
    if (!device_info().ok) return no("device is not compute capability 10.x");
    return true;
}

int launch_gemm_tc(const GemmArgs& g, cudaStream_t st) {
    const DeviceInfo di = device_info();
    if (!di.ok) return fail(BI8_ERR_CUDA, "tensor-core GEMM needs a compute capability 10.x device");
    CUtensorMap ma, mb;
    int rc = make_operand_map(&ma, g.A, g.M, g.K, g.lda, kBM);
    if (rc != BI8_OK) return rc;
    rc = make_operand_map(&mb, g.Bt, g.N, g.K, g.ldb, kBN);
    if (rc != BI8_OK) return rc;
    TcParams p;
    std::memset(&p, 0, sizeof(p));
    p.sA = g.sA;
    p.sB = g.sB;
    p.bias = g.bias;
    p.C = g.C;
    p.partials = g.partials;
    p.status = device_status_ptr();
    if (!p.status) return BI8_ERR_CUDA;
    p.ldc = g.ldc;
    p.M = (int)g.M;
    p.N = (int)g.N;
    p.K = (int)g.K;
    p.nb = (int)((g.K + g.block - 1) / g.block);
    p.tiles_m = (int)((g.M + kBM - 1) / kBM);
    p.tiles_n = (int)((g.N + kBN - 1) / kBN);
    p.out_dtype = g.out_dtype;
    p.bias_dtype = g.bias_dtype;
    const int esz = g.out_dtype == BI8_F32 ? 4 : 2;
    p.vec_store = (g.C != nullptr && aligned(g.C, 16) && (g.ldc * esz) % 16 == 0) ? 1 : 0;
    p.vec_scales = (g.partials == nullptr && aligned(g.sA, 16) && aligned(g.sB, 16) && g.M % 4 == 0 && g.N % 4 == 0) ? 1 : 0;
    const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
    if (tiles >= (1ll << 31) / 32) return fail(BI8_ERR_SHAPE, "too many output tiles");
    const bool partials = g.partials != nullptr;
    SplitPlan pl;
    pl.stages_per_split = (int)((g.K + kBK - 1) / kBK);
    if (!partials) {
        const SplitPlan want = plan_split(g.M, g.N, g.K, di.sms);
        // without a large enough, 16-byte aligned workspace the GEMM simply runs unsplit
        if (want.ksplit > 1 && g.workspace != nullptr && g.workspace_bytes >= want.bytes && aligned(g.workspace, 16)) pl = want;
    }
    p.ksplit = pl.ksplit;
    p.stages_per_split = pl.stages_per_split;
    p.ws = static_cast<float*>(g.workspace);
    const int64_t items = tiles * pl.ksplit;
    const int grid = (int)(items < di.sms ? items : di.sms);
    const bool seed = (g.flags & BI8_GEMM_NO_SEED) == 0;
    switch (g.block) {
        case 32: rc = launch_qb<32>(ma, mb, p, grid, partials, seed, st); break;
        case 64: rc = launch_qb<64>(ma, mb, p, grid, partials, seed, st); break;
        case 128: rc = launch_qb<128>(ma, mb, p, grid, partials, seed, st); break;
        default: return fail(BI8_ERR_BLOCK, "tensor-core GEMM supports block 32, 64, 128 (got %d)", g.block);
    }
    if (rc != BI8_OK || pl.ksplit == 1) return rc;
    const int64_t total = g.M * g.N;
    splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(p.ws, pl.ksplit, g.bias, g.bias_dtype, g.C, g.ldc,
                                                                          g.out_dtype, (int)g.M, (int)g.N);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

int run_mma_peak_probe(int iters, float* ms, int* sm_count) {
    const DeviceInfo di = device_info();
    if (!di.ok) return fail(BI8_ERR_CUDA, "probe needs a compute capability 10.x device");
    if (iters < 16 || iters > (1 << 22)) return fail(BI8_ERR_LIMIT, "iters must be in [16, 2^22]");
    int* status = device_status_ptr();
    if (!status) return BI8_ERR_CUDA;
    const size_t smem = kABytes + kProbeN * kBK + 1024;
    BI8_CUDA_TRY(cudaFuncSetAttribute(mma_peak_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaEvent_t e0, e1;
    BI8_CUDA_TRY(cudaEventCreate(&e0));
    BI8_CUDA_TRY(cudaEventCreate(&e1));
    mma_peak_probe_kernel<<<di.sms, 128, smem>>>(iters, status);   // warm-up
    BI8_CUDA_TRY(cudaEventRecord(e0));
    mma_peak_probe_kernel<<<di.sms, 128, smem>>>(iters, status);
    BI8_CUDA_TRY(cudaEventRecord(e1));
    BI8_CUDA_TRY(cudaEventSynchronize(e1));
    BI8_CUDA_TRY(cudaEventElapsedTime(ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (sm_count) *sm_count = di.sms;
    return BI8_OK;
}

}  // namespace bi8
