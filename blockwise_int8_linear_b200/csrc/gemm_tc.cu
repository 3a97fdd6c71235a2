// Int8 block GEMM with fused dequantize on the sm_100a tensor cores.
//
// Replaces the reference kernel at triton_functions.py:69-139 (path inside the reference project):
//   P_j = A[:, jB:(j+1)B] . Bt[:, jB:(j+1)B]^T      exact int32 (line 115)
//   acc += sB[j,n] * sA[j,m] * float(P_j) / 127^2   fp32, j ascending (line 120)
//   C = cast(acc) (+ cast(bias))                    (lines 125-131)
//
// One persistent CTA per SM works on 128 x BN output tiles.  Warp roles:
//   warp 0      producer.  Per stage two TMA copies of 128-byte-swizzled K-major operand tiles (A: 128 rows, Bt: BN
//               rows, 128 K-bytes) into a ring of kStages slots, and two TMA copies of the stage's block scales (an
//               fp32 box [blocks, 128] of sA and [blocks, BN] of sB) into a ring of kScaleStages slots, all four on the
//               stage's one "full" barrier.  Scale tensors that a tensor map cannot describe (base or row length not
//               16-byte aligned) are copied with cp.async by the warp's 32 lanes instead, arriving on the same barrier.
//               The scale ring needs no barriers of its own: the promotion warps read a stage's scales only after
//               they have seen one of its accumulators complete (the MMAs were issued after the stage's barrier), and
//               the ring is deep enough that a slot is never rewritten while in use (see kScaleStages).
//   warp 1      issues tcgen05.mma kind::i8 (M128 N=BN K32): the MMAs of one quantisation block accumulate into one of
//               three s32 accumulators in tensor memory, then a commit hands that accumulator to the promotion warps.
//   warps 2-3   spare (they only take part in set-up and teardown; see the register note below)
//   warps 4..   promotion + epilogue, PW warps per tensor-memory lane quarter.  A warp owns 32 rows x BN/PW columns of
//               the tile.  Per block it reads its part of the finished accumulator in two halves (the second in flight
//               while the first is folded), re-seeds what it has read, folds the values into fp32 accumulators in
//               registers and releases the accumulator.  After the last block of a tile it casts, adds bias and writes
//               its 32 x BN/PW part into a staging area in shared memory, from where one TMA store (or, for
//               destinations a tensor map cannot describe, a loop of coalesced stores) moves it out.
// What bounds the kernel: the fold costs two FMAs per element and block (t = P*s_row, acc += s_col*t), 2*128*BN FMAs per
// block on 128 FMA lanes = 320 cycles for BN = 160, twice the 163 cycles the MMAs of a 64-deep block need.  On top of
// that every promotion warp reads its BN/PW column scales of every block from shared memory as broadcast loads, which
// deliver 8 bytes per wavefront: 16 warps x ~21 wavefronts, plus the 144 wavefronts in which the tensor core reads the
// block's operands, is ~520 shared-memory wavefronts per block on a pipe that serves one per cycle.  Measured (block 64)
// the kernel needs ~790 cycles per block with the instruction issue slots 57 % and the shared-memory pipe 65 % busy.
//
// Registers: a scheduler (SM sub-partition) owns a quarter of the register file and every fourth warp, and setmaxnreg can
// only move registers between warps of the same scheduler.  Each scheduler has exactly one of warps 0-3, which shrinks,
// and PW promotion warps, which grow: PW = 4: 96 at launch -> 32 / 112; PW = 3: 128 -> 32 / 160; PW = 2: 168 -> 40 / 232.
//
// Seeded conversion (default): the promotion warps refill a drained accumulator with the bit pattern of 1.5*2^23 and
// every MMA accumulates on top of it.  Integer addition on that pattern is exact float arithmetic while |P| < 2^22
// (127^2 * 128 < 2^22), so the word read back is the float 1.5*2^23 + P and
//   t = fma(word, s, -1.5*2^23 * s) = fl(P * s)
// needs no int->float conversion.  s = sA[j,m]/127^2 rounded to 22 significant bits makes 1.5*2^23*s exact.
#include "bi8_common.cuh"
#include "tc_common.cuh"

#include <cstring>
#include <type_traits>


namespace bi8 {
namespace {

using namespace ptx;

constexpr int kBM = 128;                 // tile rows
constexpr int kAccBufs = 3;              // s32 accumulators in tensor memory
constexpr int kProbeN = 256;             // N of the issue-rate probe's MMAs
constexpr int kStages = 4;               // operand stages of 128 K-bytes in flight
// Scale ring depth.  The producer fills the slot of stage s after the MMA warp has committed stage s - kStages, whose last
// block was issued into an accumulator that the promotion warps had released three blocks earlier: with 2 blocks per
// stage they are then done with every stage up to s - kStages - 2, with 1 block per stage up to s - kStages - 3, with 4
// up to s - kStages - 1.  A ring of kStages + 3 slots is therefore never overwritten while a promotion warp reads it.
constexpr int kScaleStages = 8;
static_assert(kScaleStages >= kStages + 3, "scale ring too shallow for the lag of the promotion warps");
constexpr int kRoleWarps = 4;            // producer, MMA issuer, two spare: one warp per scheduler gives its registers away
constexpr uint32_t kABytes = kBM * kBK;  // 16 KiB
constexpr uint32_t kSeedBits = 0x4B400000u;   // float 1.5 * 2^23
constexpr float kSeedF = 12582912.0f;

// Geometry that depends on the number of promotion warps per lane quarter.
template <int PW>
struct Cfg {
    static_assert(PW == 2 || PW == 3 || PW == 4, "2, 3 or 4 promotion warps per lane quarter");
    static constexpr int BN = PW == 3 ? 144 : 160;        // tile columns: kAccBufs * BN <= 512 tensor-memory columns
    static constexpr int COLS = BN / PW;                  // columns owned by one promotion thread: 80, 48, 40
    static constexpr int H0 = PW == 2 ? 40 : 24;          // the accumulator is read as columns [0, H0) and [H0, COLS)
    static constexpr int H1 = COLS - H0;                  // 40, 24, 16
    static constexpr int EPI_WARPS = 4 * PW;
    static constexpr int THREADS = (kRoleWarps + EPI_WARPS) * 32;
    static constexpr int LAUNCH_REGS = PW == 2 ? 168 : PW == 3 ? 128 : 96;     // 65536 / THREADS, rounded down to a multiple of 8
    static constexpr int ROLE_REGS = PW == 2 ? 40 : 32;
    static constexpr int EPI_REGS = PW == 2 ? 232 : PW == 3 ? 160 : 112;
    static constexpr uint32_t B_BYTES = BN * kBK;
    static constexpr uint32_t STAGE_BYTES = kABytes + B_BYTES;
    static constexpr uint32_t scale_off = kStages * STAGE_BYTES;
    // setmaxnreg moves registers inside a scheduler's share of the CTA's launch-time allocation: the total after the
    // moves must not exceed it, or setmaxnreg.inc blocks forever.  (The launcher also checks the register count the
    // compiler really chose for the kernel.)
    static_assert(ROLE_REGS + PW * EPI_REGS <= (1 + PW) * LAUNCH_REGS, "register budget of a scheduler exceeds its launch allocation");
    static_assert((1 + PW) * 32 * LAUNCH_REGS <= 16384, "launch allocation exceeds a scheduler's register file");
    static_assert(kAccBufs * BN <= 512 && COLS % 8 == 0 && H0 % 8 == 0 && H1 % 8 == 0 && BN % 16 == 0, "tile geometry");
    __host__ __device__ static constexpr uint32_t a_off(int s) { return (uint32_t)s * STAGE_BYTES; }
    __host__ __device__ static constexpr uint32_t b_off(int s) { return a_off(s) + kABytes; }
};

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
    int tma_store;      // the output is described by the tensor map tmC: staged tiles leave by TMA stores
    int tma_scales;     // bit 0: sA is described by the tensor map tmSA, bit 1: sB by tmSB
    int ksplit;         // > 1: the K stages are divided over ksplit work items per tile (split-K)
    int stages_per_split;
    float* ws;          // split-K: fp32 partial results [ksplit, M, N]
    unsigned wait_limit_us;   // 0: default limit of the bounded waits (about two seconds)
    int skip_stage;     // >= 0: diagnostic, the producer leaves this stage of its first work item out
};

template <int QB, int PW>
struct Geo {
    using C = Cfg<PW>;
    static constexpr int BPS = kBK / QB;                        // quantisation blocks per stage
    static constexpr int MMAS = QB / 32;                        // MMAs (K = 32) per block
    static constexpr int SC_FLOATS = (BPS * (kBM + C::BN) + 31) / 32 * 32;   // scale floats per stage, [BPS][128] of sA then [BPS][BN] of sB, padded to 128 bytes
    static constexpr int SB_OFF = BPS * kBM;                    // first sB float of a stage
    static constexpr uint32_t bar_off = C::scale_off + kScaleStages * SC_FLOATS * 4;
    // barrier slots (8 bytes each)
    static constexpr int FULL_AB = 0, EMPTY_AB = kStages, ACC_FULL = 2 * kStages, ACC_EMPTY = 2 * kStages + kAccBufs,
                         NBARS = 2 * kStages + 2 * kAccBufs;
    static constexpr uint32_t misc_off = bar_off + NBARS * 8;   // tmem holder (4 B) + abort flag (4 B) + never-raised flag (4 B)
    // outputs leave through shared memory: every promotion warp stages 32 rows x COLS*2 bytes per pass
    static constexpr uint32_t OUT_WARP_BYTES = 32 * C::COLS * 2;
    static constexpr uint32_t out_off = (misc_off + 16 + 127) & ~127u;
    static constexpr uint32_t total = out_off + C::EPI_WARPS * OUT_WARP_BYTES;
    static_assert(OUT_WARP_BYTES % 128 == 0, "TMA store sources are 128-byte aligned");
    static_assert((SC_FLOATS * 4) % 128 == 0 && (SB_OFF * 4) % 128 == 0 && C::scale_off % 1024 == 0, "TMA destinations of the scale boxes are 128-byte aligned");
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

template <int BN>
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int& m0, int& n0) {
    // consecutive tiles (CTAs that run together) share a column panel of Bt and sweep the rows of A
    m0 = (tile % tiles_m) * kBM;
    n0 = (tile / tiles_m) * BN;
}

// Bounded wait of a converged warp: one poll by every lane, then (phase not complete yet, or the lanes disagree) the
// bounded loop.  The result is the same in all lanes, so a warp-aligned instruction after the wait is never reached by
// only some of them.  (Not a function call: the callers run under different setmaxnreg budgets.)
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, uint32_t abort_flag, long long limit) {
    if (__builtin_expect(__all_sync(0xffffffffu, mbar_test(bar, parity)), 1)) return true;
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, limit));
}

// NC (a multiple of 8, at most 40) consecutive accumulator columns of this thread's lane -> registers.
template <int NC>
__device__ __forceinline__ void tmem_load_cols(uint32_t taddr, uint32_t (&S)[NC]) {
    static_assert(NC == 40 || NC == 32 || NC == 24 || NC == 16 || NC == 8, "supported part widths");
    if constexpr (NC == 32) {
        tmem_ld32(taddr, S);
    } else if constexpr (NC == 8) {
        tmem_ld8(taddr, S);
    } else if constexpr (NC == 40) {
        tmem_ld32(taddr, reinterpret_cast<uint32_t(&)[32]>(S[0]));
        tmem_ld8(taddr + 32u, reinterpret_cast<uint32_t(&)[8]>(S[32]));
    } else if constexpr (NC == 24) {
        tmem_ld16(taddr, reinterpret_cast<uint32_t(&)[16]>(S[0]));
        tmem_ld8(taddr + 16u, reinterpret_cast<uint32_t(&)[8]>(S[16]));
    } else {
        tmem_ld16(taddr, reinterpret_cast<uint32_t(&)[16]>(S[0]));
    }
}

// Blocks go round the kAccBufs = 3 accumulators and every stage has BPS blocks, so block `blk` of the stage at position
// `rot` in a cycle of three stages is block rot*BPS + blk of that cycle and uses accumulator (rot*BPS + blk) % 3.  A
// cycle of three stages ends where it began, on accumulator 0.
template <int BPS>
struct RotInfo {
    __host__ __device__ static constexpr int buf(int rot, int blk) { return (rot * BPS + blk) % kAccBufs; }
};

// A value the compiler must treat as unknown from here on.  Loop-invariant addresses of the promotion loop go through
// this: left alone, the compiler recomputes them (from the warp index, the thread index, the shared-memory base ...)
// inside every block instead of keeping a register, which costs more instructions than the fold itself has to spare.
__device__ __forceinline__ uint32_t keep(uint32_t v) {
    asm volatile("" : "+r"(v));
    return v;
}

// Folds NC s32 words a thread has read from an accumulator (its row, columns C0 .. C0+NC-1 of its COLS, one quantisation
// block) into its fp32 accumulators: acc[n] += sB[n] * (P[n] * s), both products as packed FMAs on column pairs (PACK1
// false: the first one as scalar FMAs).  `sw` is the shared address of the block's column scales of this thread (16-byte
// aligned).
template <bool SEED, bool PACK1, int C0, int NC, int COLS>
__device__ __forceinline__ void fold_columns(const uint32_t (&S)[NC], uint32_t sw, float sxd, float negc, uint64_t (&acc2)[COLS / 2]) {
    const uint64_t sxd2 = pack_f32x2(sxd, sxd), negc2 = pack_f32x2(negc, negc);
#pragma unroll
    for (int q = 0; q < NC / 4; ++q) {
        uint64_t w0, w1, t0, t1;
        lds_2xb64(sw + (uint32_t)((C0 / 4 + q) * 16), w0, w1);
        if (SEED && PACK1) {
            t0 = fma_f32x2(pack_u32x2(S[4 * q], S[4 * q + 1]), sxd2, negc2);
            t1 = fma_f32x2(pack_u32x2(S[4 * q + 2], S[4 * q + 3]), sxd2, negc2);
        } else {
            float t[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (SEED) t[u] = __fmaf_rn(__uint_as_float(S[4 * q + u]), sxd, negc);
                else t[u] = __fmul_rn((float)(int32_t)S[4 * q + u], sxd);
            }
            t0 = pack_f32x2(t[0], t[1]);
            t1 = pack_f32x2(t[2], t[3]);
        }
        acc2[C0 / 2 + 2 * q] = fma_f32x2(w0, t0, acc2[C0 / 2 + 2 * q]);
        acc2[C0 / 2 + 2 * q + 1] = fma_f32x2(w1, t1, acc2[C0 / 2 + 2 * q + 1]);
    }
}

template <int QB, int MODE, bool SEED, int PW>
__global__ void __launch_bounds__(Cfg<PW>::THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmSA, const __grid_constant__ CUtensorMap tmSB,
               const __grid_constant__ CUtensorMap tmC, const TcParams p) {
    using C = Cfg<PW>;
    using G = Geo<QB, PW>;
    constexpr int BN = C::BN, COLS = C::COLS, H0 = C::H0, H1 = C::H1;
    constexpr bool kScales = (MODE == 0);           // the partial-sum dump uses no scales
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    // dynamic shared memory is only guaranteed 16-byte aligned: round up to the swizzle atom
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_dyn + (base - raw);
    const float* sc_ring = reinterpret_cast<const float*>(base_ptr + C::scale_off);
    const uint32_t sc_ring_u32 = base + C::scale_off;
    const uint32_t bars = base + G::bar_off;
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(base_ptr + G::misc_off);
    const uint32_t abort_flag = base + G::misc_off + 4;
    const uint32_t never_flag = base + G::misc_off + 8;
    auto bar = [&](int slot) -> uint32_t { return bars + 8u * (uint32_t)slot; };

    // the warp index through a shuffle: known to be the same in all lanes, so what is derived from it lives in uniform registers
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int nks = (p.K + kBK - 1) / kBK;
    const int num_items = num_tiles * p.ksplit;
    // limit of the bounded waits in SM cycles: about two seconds, or the diagnostic's shorter one.  The MMA warp's waits
    // get the limit itself and all others four times as much, so that a missing operand stage is reported by the wait
    // that misses it and not by a warp that starves behind it.
    const long long wait_limit_mma = p.wait_limit_us ? (long long)p.wait_limit_us * 2000ll : 4000000000ll;
    const long long wait_limit = p.wait_limit_us ? 4 * wait_limit_mma : wait_limit_mma;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            // the lane that issues the TMA copies; with scales copied by cp.async, every lane of the producer warp as well
            mbar_init(bar(G::FULL_AB + s), (kScales && p.tma_scales != 3) ? 33 : 1);
            mbar_init(bar(G::EMPTY_AB + s), 1);
        }
        for (int b = 0; b < kAccBufs; ++b) {
            mbar_init(bar(G::ACC_FULL + b), 1);
            mbar_init(bar(G::ACC_EMPTY + b), C::EPI_WARPS);
        }
        sts_u32(abort_flag, 0u);
        sts_u32(never_flag, 0u);                     // a flag nobody raises, for waits that must not be cut short
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_holder), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp < kRoleWarps) {
        setmaxnreg_dec<C::ROLE_REGS>();
        // Whole warps run the producer and MMA loops convergently and one lane issues: lanes parked at the final
        // barrier while a sibling lane loops make that loop crawl.
        if (warp == 0) {
            // ---------------- producer: operand tiles and block scales ----------------
            int stage = 0, sslot = 0;
            uint32_t phase = 0;
            int last_parity[kStages];
#pragma unroll
            for (int s = 0; s < kStages; ++s) last_parity[s] = -1;
            bool ok = true;
            bool first_item = true;
            constexpr uint32_t kSaBytes = (uint32_t)(G::BPS * kBM * 4), kSbBytes = (uint32_t)(G::BPS * BN * 4);
            const bool tma_sa = kScales && (p.tma_scales & 1), tma_sb = kScales && (p.tma_scales & 2);
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                int tile, split, ks0, ks1, m0, n0;
                item_range(item, num_tiles, nks, p.stages_per_split, tile, split, ks0, ks1);
                tile_coords<BN>(tile, p.tiles_m, m0, n0);
                for (int ks = ks0; ks < ks1; ++ks) {
                    ok = warp_wait(bar(G::EMPTY_AB + stage), phase ^ 1u, abort_flag, wait_limit);
                    if (!ok) {
                        if (lane == 0) report_timeout(p.status, abort_flag, W_EMPTY_AB);
                        break;
                    }
                    const bool skip = first_item && p.skip_stage >= 0 && ks - ks0 == p.skip_stage;   // diagnostic only
                    const uint32_t fb = bar(G::FULL_AB + stage);
                    const uint32_t sdst = sc_ring_u32 + (uint32_t)(sslot * G::SC_FLOATS * 4);
                    if (lane == 0 && !skip) {
                        mbar_expect_tx(fb, C::STAGE_BYTES + (tma_sa ? kSaBytes : 0u) + (tma_sb ? kSbBytes : 0u));
                        tma_load_2d(base + C::a_off(stage), &tmA, fb, ks * kBK, m0);
                        tma_load_2d(base + C::b_off(stage), &tmB, fb, ks * kBK, n0);
                        // boxes [BPS, 128] of sA and [BPS, BN] of sB; rows and blocks outside the tensors read as zero
                        if (tma_sa) tma_load_2d(sdst, &tmSA, fb, m0, ks * G::BPS);
                        if (tma_sb) tma_load_2d(sdst + (uint32_t)(G::SB_OFF * 4), &tmSB, fb, n0, ks * G::BPS);
                    }
                    if (kScales && !(tma_sa && tma_sb) && !skip) {
                        // A scale tensor whose rows are not 16-byte aligned: asynchronous 4-byte copies by the 32 lanes (the
                        // warp does not wait for the data; each lane's arrival on the stage's barrier fires when its
                        // copies have landed)
#pragma unroll
                        for (int blk = 0; blk < G::BPS; ++blk) {
                            const int j = ks * G::BPS + blk;
                            if (!tma_sa) {
                                const float* row = p.sA + (int64_t)j * p.M + m0;
#pragma unroll
                                for (int c = lane; c < kBM; c += 32) {
                                    const bool live = j < p.nb && m0 + c < p.M;
                                    cp_async_4(sdst + (uint32_t)((blk * kBM + c) * 4), live ? row + c : p.sA, live ? 4u : 0u);
                                }
                            }
                            if (!tma_sb) {
                                const float* row = p.sB + (int64_t)j * p.N + n0;
#pragma unroll
                                for (int c = lane; c < BN; c += 32) {
                                    const bool live = j < p.nb && n0 + c < p.N;
                                    cp_async_4(sdst + (uint32_t)((G::SB_OFF + blk * BN + c) * 4), live ? row + c : p.sB, live ? 4u : 0u);
                                }
                            }
                        }
                        cp_async_arrive(fb);
                    }
                    __syncwarp();
                    if (!skip) {
#pragma unroll
                        for (int s = 0; s < kStages; ++s)
                            if (s == stage) last_parity[s] = (int)phase;
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    if (++sslot == kScaleStages) sslot = 0;
                }
                first_item = false;
            }
            if (!ok) {
                // do not leave while our own copies may still land in this CTA's shared memory
#pragma unroll
                for (int s = 0; s < kStages; ++s)
                    if (last_parity[s] >= 0) (void)mbar_wait(bar(G::FULL_AB + s), (uint32_t)last_parity[s], never_flag, 200000000ll);
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            // Every stage has BPS blocks (blocks past the end of K multiply zero-filled operands) and the blocks go
            // round the three accumulators.  Every tile starts on accumulator 0, so which accumulator a block uses
            // depends only on the stage's position in a cycle of three stages: the K loop runs in such cycles, with the
            // stage body in three copies that have the accumulator as a constant (RotInfo) and no dispatch between
            // them.  The barrier parity of each accumulator flips with every use.
            constexpr uint32_t idesc = umma_idesc_i8(kBM, BN);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t accpar[kAccBufs] = {0u, 0u, 0u};
            bool ok = true;
            auto issue_stage = [&](auto rot_tag) {
                constexpr int ROT = decltype(rot_tag)::value;
                ok = warp_wait(bar(G::FULL_AB + stage), phase, abort_flag, wait_limit_mma);
                if (!ok) {
                    if (lane == 0) report_timeout(p.status, abort_flag, W_FULL_AB);
                    return;
                }
                tc_fence_after();
                const uint64_t adesc = umma_desc_k_sw128(base + C::a_off(stage));
                const uint64_t bdesc = umma_desc_k_sw128(base + C::b_off(stage));
#pragma unroll
                for (int blk = 0; blk < G::BPS; ++blk) {
                    const int buf = RotInfo<G::BPS>::buf(ROT, blk);
                    ok = warp_wait(bar(G::ACC_EMPTY + buf), accpar[buf], abort_flag, wait_limit_mma);
                    if (!ok) {
                        if (lane == 0) report_timeout(p.status, abort_flag, W_ACC_EMPTY);
                        return;
                    }
                    accpar[buf] ^= 1u;
                    tc_fence_after();
                    if (lane == 0) {
#pragma unroll
                        for (int i = 0; i < G::MMAS; ++i) {
                            const uint64_t koff = (uint64_t)((blk * G::MMAS + i) * 32 / 16);
                            mma_i8(tmem_base + (uint32_t)(buf * BN), adesc + koff, bdesc + koff, idesc, (SEED || i > 0) ? 1u : 0u);
                        }
                        tc_commit(bar(G::ACC_FULL + buf));
                    }
                    __syncwarp();
                }
                if (lane == 0) tc_commit(bar(G::EMPTY_AB + stage));
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            };
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                int tile, split, ks0, ks1;
                item_range(item, num_tiles, nks, p.stages_per_split, tile, split, ks0, ks1);
                for (int ks = ks0; ks < ks1 && ok; ks += 3) {
                    issue_stage(std::integral_constant<int, 0>{});
                    if (ks + 1 < ks1 && ok) issue_stage(std::integral_constant<int, 1>{});
                    if (ks + 2 < ks1 && ok) issue_stage(std::integral_constant<int, 2>{});
                }
            }
        }
    } else {
        // ---------------- promotion + epilogue ----------------
        setmaxnreg_inc<C::EPI_REGS>();
        const int quarter = warp & 3;                     // tensor-memory lanes 32*quarter .. +31 belong to this warp
        const int slice = (warp - kRoleWarps) >> 2;       // columns COLS*slice .. of the tile
        const int row = quarter * 32 + lane;
        const uint32_t t_lane = keep(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(slice * COLS));
        // eight spare tensor-memory columns of this warp's lanes keep the seed pattern
        static_assert(kAccBufs * BN + 8 * PW <= 512, "no spare tensor-memory columns for the seed pattern");
        const uint32_t t_seed = keep(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(kAccBufs * BN + 8 * slice));
        // shared addresses of this thread's row scale and of its first column scale in scale stage 0, block 0
        const uint32_t sa_addr = keep(sc_ring_u32 + (uint32_t)(row * 4));
        const uint32_t sw_addr = keep(sc_ring_u32 + (uint32_t)((G::SB_OFF + slice * COLS) * 4));
        const uint32_t bar0 = keep(bars);
        const uint32_t leader = keep(lane == 0 ? 1u : 0u);
        const float div = 1.0f / (127.0f * 127.0f);
        uint32_t seedv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) seedv[i] = kSeedBits;

        if (SEED) {
#pragma unroll
            for (int b = 0; b < kAccBufs; ++b)
#pragma unroll
                for (int c = 0; c < COLS / 8; ++c) tmem_st8(t_lane + (uint32_t)(b * BN + c * 8), seedv);
            tmem_wait_st();
            // The promotion loop re-reads the seed pattern from the spare columns in every block: the result of a load is
            // a tuple of consecutive registers, which is what the stores want, and it is live for half a block only.
            // Eight constants would be rebuilt with eight moves in front of every store; a tuple kept across the loop
            // costs eight registers that the loop does not have, and the compiler then copies it around.
            tmem_st8(t_seed, seedv);
            tmem_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < kAccBufs; ++b) mbar_arrive(bar(G::ACC_EMPTY + b));
        }
        auto reseed = [&](uint32_t taddr, int c0, int nc) {
            if (SEED) {
#pragma unroll
                for (int c = 0; c < nc / 8; ++c) tmem_st8(taddr + (uint32_t)(c0 + c * 8), seedv);
            }
        };

        int sstage = 0;
        uint32_t accpar[kAccBufs] = {0u, 0u, 0u};   // barrier parities of the three accumulators, flipped with every use
        uint32_t sc_off = 0;                      // byte offset of scale stage `sstage`
        bool ok = true;
        int fail_code = 0;

        // the tile's COLS fp32 accumulators of this thread, kept as packed pairs for fma.rn.f32x2
        uint64_t acc2[COLS / 2];
        int m = 0, nbase = 0;
        uint32_t S0[H0], S1[H1];

        // One stage of the promotion: BPS blocks.  `rot_tag` is the stage's position in a cycle of three stages, which
        // fixes the accumulator of each of its blocks (RotInfo); `ks` is the stage's index along K.
        auto promote_stage = [&](auto rot_tag, int ks) {
            constexpr int ROT = decltype(rot_tag)::value;
            using R = RotInfo<G::BPS>;
#pragma unroll
            for (int blk = 0; blk < G::BPS; ++blk) {
                const int buf = R::buf(ROT, blk);
                const uint32_t t_acc = t_lane + (uint32_t)(buf * BN);
                ok = warp_wait(bar0 + 8u * (uint32_t)(G::ACC_FULL + buf), accpar[buf], abort_flag, wait_limit);
                if (!ok) {
                    fail_code = W_ACC_FULL;
                    return;
                }
                accpar[buf] ^= 1u;
                tc_fence_after();
                if (MODE == 1) {
                    const int j = ks * G::BPS + blk;
#pragma unroll
                    for (int c = 0; c < COLS / 8; ++c) {
                        uint32_t pv[8];
                        tmem_ld8(t_acc + (uint32_t)(c * 8), pv);
                        tmem_wait_ld();
                        reseed(t_acc, c * 8, 8);
                        if (m < p.M && j < p.nb) {
                            int32_t* dst = p.partials + ((int64_t)j * p.M + m) * p.N + nbase + c * 8;
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if (nbase + c * 8 + i < p.N)
                                    dst[i] = SEED ? (int32_t)(pv[i] - kSeedBits) : (int32_t)pv[i];
                        }
                    }
                } else {
                    tmem_load_cols<H0>(t_acc, S0);
                    if (SEED) tmem_ld8(t_seed, seedv);      // the seed tuple for this block's stores
                    // the row's scale, while the read of the first half is in flight
                    float sxd = __fmul_rn(lds_f32(sa_addr + sc_off + (uint32_t)(blk * kBM * 4)), div);
                    float negc = 0.0f;
                    if (SEED) {
                        sxd = __uint_as_float((__float_as_uint(sxd) + 2u) & 0xFFFFFFFCu);   // 22 significant bits
                        negc = -__fmul_rn(kSeedF, sxd);                                      // exact
                    }
                    const uint32_t sw = sw_addr + sc_off + (uint32_t)(blk * BN * 4);
                    tmem_wait_ld();
                    tmem_load_cols<H1>(t_acc + (uint32_t)H0, S1);    // second half, in flight during the fold of the first
                    reseed(t_acc, 0, H0);
                    fold_columns<SEED, true, 0, H0, COLS>(S0, sw, sxd, negc, acc2);
                    tmem_wait_ld();
                    reseed(t_acc, H0, H1);
                    fold_columns<SEED, true, H0, H1, COLS>(S1, sw, sxd, negc, acc2);
                }
                if (SEED) tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (leader) mbar_arrive(bar0 + 8u * (uint32_t)(G::ACC_EMPTY + buf));
            }
            if (kScales) {
                sc_off += (uint32_t)(G::SC_FLOATS * 4);
                if (++sstage == kScaleStages) { sstage = 0; sc_off = 0; }
            }
        };

        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            int tile, split, ks0, ks1, m0, n0;
            item_range(item, num_tiles, nks, p.stages_per_split, tile, split, ks0, ks1);
            tile_coords<BN>(tile, p.tiles_m, m0, n0);
            m = m0 + row;
            nbase = n0 + slice * COLS;
#pragma unroll
            for (int i = 0; i < COLS / 2; ++i) acc2[i] = 0ull;

            // cycles of three stages; every tile starts on accumulator 0, like the MMA issuer
            for (int ks = ks0; ks < ks1 && ok; ks += 3) {
                promote_stage(std::integral_constant<int, 0>{}, ks);
                if (ks + 1 < ks1 && ok) promote_stage(std::integral_constant<int, 1>{}, ks + 1);
                if (ks + 2 < ks1 && ok) promote_stage(std::integral_constant<int, 2>{}, ks + 2);
            }
            if (!ok) break;

            if (MODE == 0) {
                // The tile leaves through the warp's staging area in shared memory: every lane writes its row's share
                // (ROWB bytes), then either one TMA store or a loop of coalesced stores moves the 32 x ROWB bytes out.
                // 2-byte outputs take one pass of COLS columns, 4-byte outputs (fp32, split-K partial sums) two passes of
                // COLS / 2.  Addresses are derived here from the thread index rather than kept in registers through the
                // K loop, whose register budget is full.
                constexpr uint32_t ROWB = (uint32_t)(COLS * 2);
                uint32_t tid_now;
                asm volatile("mov.u32 %0, %%tid.x;" : "=r"(tid_now));
                const uint32_t ln = tid_now & 31u;
                const uint32_t out_stage = base + G::out_off + ((tid_now >> 5) - (uint32_t)kRoleWarps) * G::OUT_WARP_BYTES;
                const uint32_t my_row = out_stage + ln * ROWB;
                const bool partial = p.ksplit > 1;
                const bool wide = partial || p.out_dtype == BI8_F32;
                const bool bf = p.out_dtype == BI8_BF16;
                const bool has_bias = p.bias != nullptr && !partial;   // split-K: cast and bias happen in the reduction
                const int row0 = m - (int)ln;                         // first row of the warp's part
                auto bias_at = [&](int n) -> float {
                    if (n >= p.N) return 0.0f;
                    if (p.bias_dtype == BI8_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
                    if (p.bias_dtype == BI8_F16) return __half2float(static_cast<const __half*>(p.bias)[n]);
                    return static_cast<const float*>(p.bias)[n];
                };
                const int passes = wide ? 2 : 1;
#pragma unroll 1
                for (int ps = 0; ps < passes; ++ps) {
                    const int col0 = nbase + ps * (COLS / 2);
                    // the previous TMA store must have read the staging area before it is written again
                    if (p.tma_store && ln == 0) tma_store_wait_read();
                    __syncwarp();
                    if (wide) {
#pragma unroll
                        for (int g = 0; g < COLS / 8; ++g) {
                            float v[4];
                            unpack_f32x2(acc2[2 * g], v[0], v[1]);
                            unpack_f32x2(acc2[2 * g + 1], v[2], v[3]);
                            if (has_bias) {
#pragma unroll
                                for (int u = 0; u < 4; ++u) v[u] = __fadd_rn(v[u], bias_at(col0 + g * 4 + u));
                            }
                            sts_v4(my_row + (uint32_t)(g * 16), __float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]),
                                   __float_as_uint(v[3]));
                        }
                        // the second pass finds its columns where the first found its own
#pragma unroll
                        for (int i = 0; i < COLS / 4; ++i) acc2[i] = acc2[i + COLS / 4];
                    } else {
#pragma unroll
                        for (int g = 0; g < COLS / 8; ++g) {
                            uint32_t w[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                float lo, hi;
                                unpack_f32x2(acc2[g * 4 + u], lo, hi);
                                uint32_t pk = bf ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
                                if (has_bias) {
                                    // the reference adds the bias after the cast, in the output type (lines 127-131)
                                    const int n = col0 + g * 8 + 2 * u;
                                    const float blo = bias_at(n), bhi = bias_at(n + 1);
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
                            sts_v4(my_row + (uint32_t)(g * 16), w[0], w[1], w[2], w[3]);
                        }
                    }
                    if (p.tma_store) {
                        // rows and columns of the box that lie outside the tensor are not written
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (ln == 0 && col0 < p.N && row0 < p.M) {
                            tma_store_2d(&tmC, out_stage, col0, row0);
                            tma_store_commit();
                        }
                    } else {
                        // Destinations that a tensor map cannot describe (base or row pitch not 16-byte aligned) and
                        // split-K partial sums: consecutive lanes store consecutive 4-byte words of a row, or 2-byte
                        // elements where the rows of a 16-bit output are not all 4-byte aligned.
                        __syncwarp();
                        const int esz = wide ? 4 : 2;
                        unsigned char* dst;
                        int64_t pitch;
                        if (partial) {
                            pitch = (int64_t)p.N * 4;
                            dst = reinterpret_cast<unsigned char*>(p.ws) + ((int64_t)split * p.M + row0) * pitch + (int64_t)col0 * 4;
                        } else {
                            pitch = p.ldc * esz;
                            dst = static_cast<unsigned char*>(p.C) + (int64_t)row0 * pitch + (int64_t)col0 * esz;
                        }
                        const int rows_valid = p.M - row0;                         // may exceed 32 or be negative
                        const int cols_left = p.N - col0;
                        const int cols_pass = wide ? COLS / 2 : COLS;
                        const int cols_valid = cols_left < cols_pass ? cols_left : cols_pass;
                        if (wide || (((reinterpret_cast<uintptr_t>(dst) | (uintptr_t)pitch) & 3u) == 0)) {
                            constexpr int WPR = (int)ROWB / 4;                     // words per staged row
                            const int words = wide ? cols_valid : (cols_valid >> 1);
                            const bool odd_tail = !wide && (cols_valid & 1) && cols_valid > 0;
#pragma unroll 4
                            for (int idx = (int)ln; idx < 32 * WPR; idx += 32) {
                                const int r = idx / WPR, w = idx - r * WPR;
                                if (r < rows_valid) {
                                    const uint32_t v = lds_u32(out_stage + (uint32_t)(idx * 4));
                                    unsigned char* d = dst + (int64_t)r * pitch + w * 4;
                                    if (w < words) *reinterpret_cast<uint32_t*>(d) = v;
                                    else if (odd_tail && w == words) *reinterpret_cast<uint16_t*>(d) = (uint16_t)(v & 0xffffu);
                                }
                            }
                        } else {
                            constexpr int EPR = (int)ROWB / 2;                     // elements per staged row
#pragma unroll 4
                            for (int idx = (int)ln; idx < 32 * EPR; idx += 32) {
                                const int r = idx / EPR, c = idx - r * EPR;
                                if (r < rows_valid && c < cols_valid)
                                    *reinterpret_cast<uint16_t*>(dst + (int64_t)r * pitch + c * 2) = lds_u16(out_stage + (uint32_t)(idx * 2));
                            }
                        }
                    }
                }
            }
        }
        // shared memory stays valid until the last store has read it
        if (lane == 0) tma_store_wait_read();
        if (!ok) {
            if (lane == 0) report_timeout(p.status, abort_flag, fail_code);
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Split-K reduction: C[m,n] = cast(sum_s ws[s,m,n]) (+ cast(bias[n]) in the output type).  The splits are added in
// ascending order, so the result does not depend on scheduling.  VEC = 4: a thread takes four consecutive columns of a row
// (16-byte loads of every split, all in flight before the first addition); VEC = 1 for N not a multiple of 4.
template <int VEC>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ ws, int ksplit, const void* __restrict__ bias,
                                                            int bias_dtype, void* __restrict__ C, int64_t ldc, int out_dtype,
                                                            int M, int N) {
    const int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * VEC;
    const int64_t total = (int64_t)M * N;
    if (i >= total) return;
    const int m = (int)(i / N), n = (int)(i % N);
    float acc[VEC];
#pragma unroll
    for (int u = 0; u < VEC; ++u) acc[u] = 0.0f;
    for (int s0 = 0; s0 < ksplit; s0 += 4) {
        float v[4][VEC];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (s0 + q < ksplit) {
                const float* src = ws + (int64_t)(s0 + q) * total + i;
                if (VEC == 4) {
                    const float4 f = __ldcg(reinterpret_cast<const float4*>(src));
                    v[q][0] = f.x;
                    if (VEC > 1) { v[q][1 % VEC] = f.y; v[q][2 % VEC] = f.z; v[q][3 % VEC] = f.w; }
                } else {
                    v[q][0] = __ldcg(src);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (s0 + q < ksplit) {
#pragma unroll
                for (int u = 0; u < VEC; ++u) acc[u] = __fadd_rn(acc[u], v[q][u]);
            }
    }
    const bool hb = bias != nullptr;
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
        float bv = 0.0f;
        if (hb) {
            if (bias_dtype == BI8_BF16) bv = __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n + u]);
            else if (bias_dtype == BI8_F16) bv = __half2float(static_cast<const __half*>(bias)[n + u]);
            else bv = static_cast<const float*>(bias)[n + u];
        }
        const int64_t o = (int64_t)m * ldc + n + u;
        if (out_dtype == BI8_F32) {
            static_cast<float*>(C)[o] = hb ? __fadd_rn(acc[u], bv) : acc[u];
        } else if (out_dtype == BI8_BF16) {
            __nv_bfloat16 c = __float2bfloat16_rn(acc[u]);
            if (hb) c = __float2bfloat16_rn(__fadd_rn(__bfloat162float(c), __bfloat162float(__float2bfloat16_rn(bv))));
            static_cast<__nv_bfloat16*>(C)[o] = c;
        } else {
            __half c = __float2half_rn(acc[u]);
            if (hb) c = __float2half_rn(__fadd_rn(__half2float(c), __half2float(__float2half_rn(bv))));
            static_cast<__half*>(C)[o] = c;
        }
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

struct TcMaps {
    CUtensorMap a, b, sa, sb, c;
};

template <int QB, int MODE, bool SEED, int PW>
int launch_one(const TcMaps& tm, const TcParams& p, int grid, cudaStream_t st) {
    using C = Cfg<PW>;
    constexpr size_t smem = Geo<QB, PW>::total + 1024;
    static SmemOptIn opt_in;
    const int rc = opt_in.ensure(gemm_tc_kernel<QB, MODE, SEED, PW>, smem);
    if (rc != BI8_OK) return rc;
    // setmaxnreg.inc waits for registers that the role warps of the same scheduler give up: if the compiler gave the
    // kernel fewer registers per thread than the budget was written for, the wait would never end.  Checked once.
    static int regs_ok = 0;       // 0 unknown, 1 fine, -1 refused
    if (regs_ok == 0) {
        cudaFuncAttributes fa;
        BI8_CUDA_TRY(cudaFuncGetAttributes(&fa, gemm_tc_kernel<QB, MODE, SEED, PW>));
        regs_ok = ((1 + PW) * fa.numRegs >= C::ROLE_REGS + PW * C::EPI_REGS && (1 + PW) * 32 * fa.numRegs <= 16384) ? 1 : -1;
    }
    if (regs_ok < 0) return fail(BI8_ERR_CUDA, "tensor-core GEMM: the kernel was compiled with a register count its register moves do not fit");
    gemm_tc_kernel<QB, MODE, SEED, PW><<<grid, C::THREADS, smem, st>>>(tm.a, tm.b, tm.sa, tm.sb, tm.c, p);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

// Promotion warps per lane quarter (and with it the tile width) of the kernel that runs.
constexpr int kPW = 4;
int tc_bn() { return Cfg<kPW>::BN; }

template <int QB>
int launch_qb(const TcMaps& tm, const TcParams& p, int grid, bool partials, bool seed, cudaStream_t st) {
    if (partials) return seed ? launch_one<QB, 1, true, kPW>(tm, p, grid, st) : launch_one<QB, 1, false, kPW>(tm, p, grid, st);
    return seed ? launch_one<QB, 0, true, kPW>(tm, p, grid, st) : launch_one<QB, 0, false, kPW>(tm, p, grid, st);
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
    const int bn = tc_bn();
    const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
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
    int dev = 0;
    BI8_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(BI8_ERR_CUDA, "device ordinal %d out of range", dev);
    const int bps = kBK / g.block;
    const int nb = (int)((g.K + g.block - 1) / g.block);
    TcMaps tm;
    int rc = cached_operand_map(&tm.a, dev, g.A, g.M, g.K, g.lda, kBM);
    if (rc != BI8_OK) return rc;
    const int bn = tc_bn();
    rc = cached_operand_map(&tm.b, dev, g.Bt, g.N, g.K, g.ldb, bn);
    if (rc != BI8_OK) return rc;
    TcParams p;
    std::memset(&p, 0, sizeof(p));
    const bool partials = g.partials != nullptr;
    // a scale tensor goes through TMA when a tensor map can describe it: 16-byte aligned base and row length
    const bool tma_sa = !partials && aligned(g.sA, 16) && g.M % 4 == 0, tma_sb = !partials && aligned(g.sB, 16) && g.N % 4 == 0;
    p.tma_scales = (tma_sa ? 1 : 0) | (tma_sb ? 2 : 0);
    tm.sa = tm.a;          // stand-ins that are never dereferenced
    tm.sb = tm.b;
    if (tma_sa) {
        rc = cached_scale_map(&tm.sa, dev, g.sA, nb, g.M, kBM, bps);
        if (rc != BI8_OK) return rc;
    }
    if (tma_sb) {
        rc = cached_scale_map(&tm.sb, dev, g.sB, nb, g.N, bn, bps);
        if (rc != BI8_OK) return rc;
    }
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
    p.nb = nb;
    p.tiles_m = (int)((g.M + kBM - 1) / kBM);
    p.tiles_n = (int)((g.N + bn - 1) / bn);
    p.out_dtype = g.out_dtype;
    p.bias_dtype = g.bias_dtype;
    const int esz = g.out_dtype == BI8_F32 ? 4 : 2;
    p.vec_store = (g.C != nullptr && aligned(g.C, 16) && (g.ldc * esz) % 16 == 0) ? 1 : 0;
    p.wait_limit_us = g.wait_limit_us;
    p.skip_stage = g.skip_stage;
    tm.c = tm.a;           // stand-in, never dereferenced without tma_store
    const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
    if (tiles >= (1ll << 31) / 32) return fail(BI8_ERR_SHAPE, "too many output tiles");
    SplitPlan pl;
    pl.stages_per_split = (int)((g.K + kBK - 1) / kBK);
    if (!partials) {
        const SplitPlan want = plan_split(g.M, g.N, g.K, di.sms);
        // without a large enough, 16-byte aligned workspace the GEMM simply runs unsplit
        if (want.ksplit > 1 && g.workspace != nullptr && g.workspace_bytes >= want.bytes && aligned(g.workspace, 16)) pl = want;
    }
    p.ksplit = pl.ksplit;
    p.stages_per_split = pl.stages_per_split;
    if (!partials && pl.ksplit == 1 && p.vec_store) {
        // one box = what a promotion warp stages per pass: 32 rows x (its columns, or half of them for 4-byte elements)
        const int cols = bn / kPW;
        rc = cached_output_map(&tm.c, dev, g.C, esz, g.M, g.N, g.ldc, 32, esz == 2 ? cols : cols / 2);
        if (rc != BI8_OK) return rc;
        p.tma_store = 1;
    }
    p.ws = static_cast<float*>(g.workspace);
    const int64_t items = tiles * pl.ksplit;
    const int grid = (int)(items < di.sms ? items : di.sms);
    const bool seed = (g.flags & BI8_GEMM_NO_SEED) == 0;
    switch (g.block) {
        case 32: rc = launch_qb<32>(tm, p, grid, partials, seed, st); break;
        case 64: rc = launch_qb<64>(tm, p, grid, partials, seed, st); break;
        case 128: rc = launch_qb<128>(tm, p, grid, partials, seed, st); break;
        default: return fail(BI8_ERR_BLOCK, "tensor-core GEMM supports block 32, 64, 128 (got %d)", g.block);
    }
    if (rc != BI8_OK || pl.ksplit == 1) return rc;
    const int64_t total = g.M * g.N;
    if (g.N % 4 == 0)
        splitk_reduce_kernel<4><<<(unsigned)((total / 4 + 255) / 256), 256, 0, st>>>(p.ws, pl.ksplit, g.bias, g.bias_dtype, g.C, g.ldc,
                                                                                 g.out_dtype, (int)g.M, (int)g.N);
    else
        splitk_reduce_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(p.ws, pl.ksplit, g.bias, g.bias_dtype, g.C, g.ldc,
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
