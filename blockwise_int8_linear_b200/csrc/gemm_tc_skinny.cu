// Int8 block GEMM with fused dequantize for few activation rows (decode and small batches: M <= 64), on the sm_100a tensor
// cores with the operand roles exchanged.
//
// Same contract as the reference kernel at triton_functions.py:69-139 (path inside the reference project).  With so few
// rows of A the work is one pass over the weights Bt[N, K]: the kernel is bound by streaming them from HBM, and is
// organised around that stream.
//   * The weights are the M operand of the MMA: a tile is 128 weight rows, the activations (padded to 16, 32 or 64
//     rows by the TMA's zero fill) are the N operand, so one tcgen05.mma kind::i8 (M128 N16..64 K32) covers 128 weight
//     rows and every activation row, and the s32 accumulator of a quantisation block is only 16..64 tensor-memory columns.
//   * All (tile, K stage) pairs form one sequence that is cut into equal contiguous ranges, one per CTA and one CTA
//     per SM, so every SM streams the same number of bytes whatever N and K are.  A range may begin or end inside a
//     tile: such a part of a tile goes to an fp32 workspace slot (at most two per CTA) and a second kernel adds the
//     slots of a tile in ascending K order; tiles that lie completely inside one range are written directly.  That
//     kernel is launched with programmatic stream serialisation: it becomes resident while this one runs and
//     griddepcontrol.wait releases it when this grid has completed.  (Adding the parts inside the GEMM, by whichever
//     CTA finishes a tile last, was measured slower than the second launch: the fence, the arrival count and the
//     read-back are three dependent trips to L2 at the end of every CTA.)
//   * Warp roles: promotion warps (four per 16 activation rows, or per 32 for 64 rows; one per tensor-memory lane
//     quarter) convert and scale;
//     one producer warp issues, per stage, three TMA copies that complete on one barrier: 128 weight rows x 128
//     K-bytes, the activation rows of the same K range, and the stage's weight scales (a [blocks, 128] fp32 box of
//     sB); two MMA issuer warps take the stages in turn (one accumulator range per quantisation block, one commit per
//     stage).
//   * With FUSED the activations arrive as bf16/fp16/fp32 and four more warps quantize, per stage, the 128 K-columns of
//     every activation row into the stage's operand tile (same arithmetic as the standalone quantizer, written in the
//     128-byte swizzle the MMA expects) and their block scales into the scale table: quantize-on-load in one kernel.
//     It is the slower of the two quantize-on-load forms; the default one is skinny_quantize_kernel in front of this
//     kernel, overlapped with its start (see the launch code at the end of the file).
//   * Promotion follows the reference's order term by term, sB*(sA*(float(P)*fl32(1/127^2))), added in ascending block
//     order within a range, so a tile that is not divided is bit-identical to the CUDA-core kernel.
#include "quant_math.cuh"
#include "tc_common.cuh"
#include "peer_common.cuh"

#include <cstring>

namespace bi8 {
namespace {

using namespace ptx;

constexpr int kTileRows = 128;    // weight rows per tile (the MMA's M)
constexpr int kSkMaxM = 64;       // beyond 64 activation rows the promotion (5 instructions per element and block, in the
                                  // reference's order) costs more than the weights take to arrive: measured slower than
                                  // the general kernel at 128 rows

constexpr int pow2_at_least(int x) {
    int p = 32;
    while (p < x) p *= 2;
    return p;
}

constexpr int kQuantWarps = 4;    // FUSED: warps that quantize the activations of a stage
constexpr int kMmaWarps = 2;      // MMA issuers, taking the stages in turn

template <int QB, int BNS, bool FUSED = false>
struct SkGeo {
    // ring depth: the loop producer -> HBM -> MMA -> promotion -> producer takes a few thousand cycles per slot, and a
    // stage should be re-issued every ~700 to keep up with HBM
    static constexpr int STAGES = BNS == 16 ? 8 : 6;
    static constexpr int BPS = kBK / QB;                  // quantisation blocks per stage
    static constexpr int MMAS = QB / 32;                  // MMAs (K = 32) per block
    static constexpr int CW = BNS <= 32 ? 16 : 32;        // activation rows (accumulator columns) per promotion warp
    static constexpr int CHUNKS = BNS / CW;
    static constexpr int PROMO_WARPS = 4 * CHUNKS;
    static constexpr int VB = CW == 16 ? BPS : 1;         // blocks whose accumulators a promotion thread loads at once
    static constexpr int THREADS = (PROMO_WARPS + 1 + kMmaWarps + (FUSED ? kQuantWarps : 0)) * 32;
    static constexpr int ACC_STRIDE = BPS * BNS;          // tensor-memory columns of one stage's accumulators
    static constexpr int NBUF = (512 / ACC_STRIDE) < 4 ? (512 / ACC_STRIDE) : 4;
    static constexpr int TMEM_COLS = pow2_at_least(NBUF * ACC_STRIDE);
    static constexpr uint32_t W_BYTES = kTileRows * kBK;
    static constexpr uint32_t X_BYTES = BNS * kBK;
    static constexpr uint32_t S_TX = BPS * kTileRows * 4;                 // bytes the scale copy delivers
    static constexpr uint32_t S_BYTES = S_TX < 1024 ? 1024 : S_TX;        // keeps every stage 1024-byte aligned
    static constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES + S_BYTES;
    static constexpr uint32_t bar_off = STAGES * STAGE_BYTES;
    static constexpr int FULL_AB = 0, EMPTY_AB = STAGES, ACC_FULL = 2 * STAGES, ACC_EMPTY = 2 * STAGES + NBUF,
                         NBARS = 2 * STAGES + 2 * NBUF;
    static constexpr uint32_t misc_off = bar_off + NBARS * 8;             // tmem holder, abort flag, never-raised flag
    static constexpr uint32_t sx_off = (misc_off + 32 + 15) & ~15u;       // activation scales [nb][BNS]
};

// dynamic shared memory of a launch: stage ring, barriers, activation scales [nb][BNS], alignment slack
template <int QB, int BNS, bool FUSED>
constexpr size_t smem_of(int nb) {
    return (size_t)SkGeo<QB, BNS, FUSED>::sx_off + (size_t)nb * BNS * 4 + 1024;
}

struct SkParams {
    const float* sA;
    const void* X;          // FUSED: activations before quantization, row pitch ldx elements
    int64_t ldx;
    int x_dtype;
    const void* bias;
    int64_t bias_ld;        // row pitch of `bias` in elements: 0 = one row for all (a bias), else an [M, N] addend (a residual)
    void* C;
    float* ws;
    int* status;
    int64_t ldc;
    long long total_stages;
    int M, N, K, nb, nks;
    int out_dtype, bias_dtype;
    int live_chunks;    // groups of CW activation rows that hold a valid row
    int early_weights;  // the weight copies of the first stages may be issued before the preceding kernel has completed
};

// first (tile, stage) pair of CTA c when `total` pairs are divided over `ctas` CTAs
__host__ __device__ __forceinline__ long long range_start(long long c, long long total, long long ctas) { return c * total / ctas; }

// C[m, n] = cast(acc) (+ cast(bias[m * bias_ld + n]) in the output type: reference lines 125-131)
__device__ __forceinline__ void finish_store(float acc, int m, int n, const void* bias, int bias_dtype, int64_t bias_ld, void* C,
                                             int64_t ldc, int out_dtype) {
    float bv = 0.0f;
    const bool hb = bias != nullptr;
    if (hb) {
        const int64_t bi = (int64_t)m * bias_ld + n;
        if (bias_dtype == BI8_BF16) bv = __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[bi]);
        else if (bias_dtype == BI8_F16) bv = __half2float(static_cast<const __half*>(bias)[bi]);
        else bv = static_cast<const float*>(bias)[bi];
    }
    const int64_t o = (int64_t)m * ldc + n;
    if (out_dtype == BI8_F32) {
        static_cast<float*>(C)[o] = hb ? __fadd_rn(acc, bv) : acc;
    } else if (out_dtype == BI8_BF16) {
        __nv_bfloat16 c = __float2bfloat16_rn(acc);
        if (hb) c = __float2bfloat16_rn(__fadd_rn(__bfloat162float(c), __bfloat162float(__float2bfloat16_rn(bv))));
        static_cast<__nv_bfloat16*>(C)[o] = c;
    } else {
        __half c = __float2half_rn(acc);
        if (hb) c = __float2half_rn(__fadd_rn(__half2float(c), __half2float(__float2half_rn(bv))));
        static_cast<__half*>(C)[o] = c;
    }
}

template <int QB, int BNS, bool FUSED>
__global__ void __launch_bounds__(SkGeo<QB, BNS, FUSED>::THREADS, 1)
gemm_tc_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                      const __grid_constant__ CUtensorMap tmS, const SkParams p) {
    using G = SkGeo<QB, BNS, FUSED>;
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;      // the swizzle atom needs 1024-byte alignment
    unsigned char* base_ptr = smem_dyn + (base - raw);
    const uint32_t bars = base + G::bar_off;
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(base_ptr + G::misc_off);
    const uint32_t abort_flag = base + G::misc_off + 4;
    const uint32_t never_flag = base + G::misc_off + 8;
    float* sx = reinterpret_cast<float*>(base_ptr + G::sx_off);
    const uint32_t sx_u32 = base + G::sx_off;
    auto bar = [&](int slot) -> uint32_t { return bars + 8u * (uint32_t)slot; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int live_warps = 4 * p.live_chunks;
    constexpr int PW = G::PROMO_WARPS, MW = G::PROMO_WARPS + 1, QW0 = G::PROMO_WARPS + 1 + kMmaWarps;
    static_assert(G::STAGES % kMmaWarps == 0 && G::NBUF % kMmaWarps == 0, "every issuer keeps its own stages and accumulators");

    const long long s_begin = range_start(blockIdx.x, p.total_stages, gridDim.x);
    const long long s_end = range_start((long long)blockIdx.x + 1, p.total_stages, gridDim.x);
    // position of the CTA's first stage; every role then steps (tile, ks) by itself, without a division per stage
    const int tile_begin = (int)(s_begin / p.nks), ks_begin = (int)(s_begin - (long long)tile_begin * p.nks);

    // one lane; `with_x` false leaves out the activation tile, whose copy then has to follow (issue_x)
    auto issue_stage = [&](int stage, int tile, int ks, bool with_x) {
        const uint32_t dst = base + (uint32_t)stage * G::STAGE_BYTES;
        mbar_expect_tx(bar(G::FULL_AB + stage), G::W_BYTES + (FUSED ? 0u : G::X_BYTES) + G::S_TX);
        tma_load_2d(dst, &tmW, bar(G::FULL_AB + stage), ks * kBK, tile * kTileRows);
        if (!FUSED && with_x) tma_load_2d(dst + G::W_BYTES, &tmX, bar(G::FULL_AB + stage), ks * kBK, 0);
        tma_load_2d(dst + G::W_BYTES + G::X_BYTES, &tmS, bar(G::FULL_AB + stage), tile * kTileRows, ks * G::BPS);
    };
    auto issue_x = [&](int stage, int ks) {
        tma_load_2d(base + (uint32_t)stage * G::STAGE_BYTES + G::W_BYTES, &tmX, bar(G::FULL_AB + stage), ks * kBK, 0);
    };

    // The producer warp sets the barriers up, tells the others (named barrier 2: it arrives, they wait, so it never stands
    // still) and starts the copies of the first stages right away: the ring is empty, nothing has to be waited for.  The
    // tensor-memory allocation runs beside it.
    int pre_tile = tile_begin, pre_ks = ks_begin, pre_count = 0;
    if (warp == PW) {
        if (lane == 0) {
            for (int s = 0; s < G::STAGES; ++s) {
                mbar_init(bar(G::FULL_AB + s), FUSED ? 1 + kQuantWarps : 1);   // the TMA's bytes (+ the quantizer warps)
                // a stage is free again when every promotion warp has seen its accumulator complete (so the MMAs have
                // read the operands) and has taken its scales
                mbar_init(bar(G::EMPTY_AB + s), live_warps);
            }
            for (int b = 0; b < G::NBUF; ++b) {
                mbar_init(bar(G::ACC_FULL + b), 1);
                mbar_init(bar(G::ACC_EMPTY + b), live_warps);
            }
            sts_u32(abort_flag, 0u);
            sts_u32(never_flag, 0u);
            mbar_fence_init();
            fence_proxy_async_smem();
        }
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"n"(G::THREADS) : "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the reduction kernel may be made resident
        // The kernel is always launched so that it may start before its predecessor in the stream has completed.  Behind
        // this library's own activation quantizer the weights are known to be at rest and their copies start at once;
        // behind any other kernel (which may be the one writing the weights) nothing is read before the wait.
        if (!p.early_weights) asm volatile("griddepcontrol.wait;" ::: "memory");
        while (pre_count < G::STAGES && s_begin + pre_count < s_end) {
            if (lane == 0) issue_stage(pre_count, pre_tile, pre_ks, false);
            ++pre_count;
            if (++pre_ks == p.nks) { pre_ks = 0; ++pre_tile; }
        }
        // Everything above touched only the weights and their scales.  The activations come from the kernel launched just
        // before this one (a quantizer that lets its dependents start early): wait for it here.
        if (p.early_weights) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (!FUSED && lane == 0) {
            int ks = ks_begin;
            for (int q = 0; q < pre_count; ++q) {
                issue_x(q, ks);
                if (++ks == p.nks) ks = 0;
            }
        }
        __syncwarp();
    }
    if (warp == MW) {
        tmem_alloc(smem_u32((const void*)tmem_holder), G::TMEM_COLS);
        tmem_relinquish();
    }
    if (warp != PW) {
        tc_fence_before();
        asm volatile("bar.sync 2, %0;" ::"n"(G::THREADS) : "memory");
        tc_fence_after();
    }
    const uint32_t tmem_base = (warp != PW) ? *tmem_holder : 0u;       // the producer never touches tensor memory

    if (warp == PW) {
        // ---------------- TMA producer ----------------
        int stage = pre_count == G::STAGES ? 0 : pre_count;
        uint32_t phase = pre_count == G::STAGES ? 1u : 0u;
        int last_parity[G::STAGES];
#pragma unroll
        for (int q = 0; q < G::STAGES; ++q) last_parity[q] = q < pre_count ? 0 : -1;
        int tile = pre_tile, ks = pre_ks;
        bool ok = true;
        for (long long s = s_begin + pre_count; s < s_end; ++s) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar(G::EMPTY_AB + stage), phase ^ 1u, abort_flag));
            if (!ok) {
                if (lane == 0) report_timeout(p.status, abort_flag, W_EMPTY_AB);
                break;
            }
            if (lane == 0) issue_stage(stage, tile, ks, true);
            __syncwarp();
#pragma unroll
            for (int q = 0; q < G::STAGES; ++q)
                if (q == stage) last_parity[q] = (int)phase;
            if (++stage == G::STAGES) { stage = 0; phase ^= 1u; }
            if (++ks == p.nks) { ks = 0; ++tile; }
        }
        if (!ok) {
            // do not leave while our own copies may still land in this CTA's shared memory
#pragma unroll
            for (int q = 0; q < G::STAGES; ++q)
                if (last_parity[q] >= 0) (void)mbar_wait(bar(G::FULL_AB + q), (uint32_t)last_parity[q], never_flag, 200000000ll);
        }
    } else if (warp >= MW && warp < MW + kMmaWarps) {
        // ---------------- MMA issuers ----------------
        // Issuing the four K = 32 MMAs of a stage and polling its two barriers costs one thread several hundred cycles, more
        // than the stage's bytes take to arrive, so kMmaWarps warps take the stages in turn (stage ring slots and
        // accumulator ranges of one residue class each).
        constexpr uint32_t idesc = umma_idesc_i8(kTileRows, BNS);
        const int me = warp - MW;
        int stage = me, buf = me, ks = ks_begin + me;
        while (ks >= p.nks) ks -= p.nks;
        uint32_t phase = 0, accphase = 0;
        for (long long s = s_begin + me; s < s_end; s += kMmaWarps) {
            // operands landed and an accumulator range is free: one vote for both
            const bool got_ab = mbar_wait(bar(G::FULL_AB + stage), phase, abort_flag);
            const bool got_acc = got_ab && mbar_wait(bar(G::ACC_EMPTY + buf), accphase ^ 1u, abort_flag);
            if (!__all_sync(0xffffffffu, got_acc)) {
                if (lane == 0) report_timeout(p.status, abort_flag, got_ab ? W_ACC_EMPTY : W_FULL_AB);
                break;
            }
            tc_fence_after();
            if (lane == 0) {
                const uint32_t st_base = base + (uint32_t)stage * G::STAGE_BYTES;
                const uint64_t wdesc = umma_desc_k_sw128(st_base);
                const uint64_t xdesc = umma_desc_k_sw128(st_base + G::W_BYTES);
#pragma unroll
                for (int blk = 0; blk < G::BPS; ++blk) {
                    if (ks * G::BPS + blk < p.nb) {
#pragma unroll
                        for (int i = 0; i < G::MMAS; ++i) {
                            const uint64_t koff = (uint64_t)((blk * G::MMAS + i) * 32 / 16);
                            mma_i8(tmem_base + (uint32_t)(buf * G::ACC_STRIDE + blk * BNS), wdesc + koff, xdesc + koff, idesc,
                                   i > 0 ? 1u : 0u);
                        }
                    }
                }
                // one commit per stage: the promotion warps release the stage's shared memory once they have seen it
                tc_commit(bar(G::ACC_FULL + buf));
            }
            __syncwarp();
            stage += kMmaWarps;
            if (stage >= G::STAGES) { stage -= G::STAGES; phase ^= 1u; }
            buf += kMmaWarps;
            if (buf >= G::NBUF) { buf -= G::NBUF; accphase ^= 1u; }
            ks += kMmaWarps;
            while (ks >= p.nks) ks -= p.nks;
        }
    } else if (FUSED && warp >= QW0) {
        // ---------------- quantize-on-load: the activations of a stage, straight into the MMA's operand tile -------------
        // A unit is 8 consecutive K elements of one activation row; a stage holds 16 units per row.  Thread t of the 128
        // takes units t, t + 128, ...: the units of one quantisation block sit in QB/8 neighbouring lanes, whose absmax is
        // an xor-shuffle reduction.  The raw values of the next stage are loaded before the current one is converted.
        constexpr int UNITS = BNS / 8;                     // units per thread and stage (BNS * 16 / 128)
        constexpr int LPB = QB / 8;                        // lanes that share a block
        const int qt = (int)threadIdx.x - QW0 * 32;
        const bool wide = p.x_dtype == BI8_F32;
        const int esz = wide ? 4 : 2;
        const unsigned char* xb = static_cast<const unsigned char*>(p.X);
        uint4 cur[UNITS][2], nxt[UNITS][2];
        asm volatile("griddepcontrol.wait;" ::: "memory");
        auto load_stage = [&](int ks, uint4 (&r)[UNITS][2]) {
#pragma unroll
            for (int u = 0; u < UNITS; ++u) {
                const int unit = qt + u * 128, m = unit >> 4, k = ks * kBK + (unit & 15) * 8;
                r[u][0] = make_uint4(0u, 0u, 0u, 0u);
                r[u][1] = make_uint4(0u, 0u, 0u, 0u);
                if (m < p.M && k < p.K) {
                    const unsigned char* src = xb + ((int64_t)m * p.ldx + k) * esz;
                    r[u][0] = ld_nc_v4(src);
                    if (wide) r[u][1] = ld_nc_v4(src + 16);
                }
            }
        };
        int stage = 0;
        uint32_t phase = 0;
        int ks = ks_begin;
        if (s_begin < s_end) load_stage(ks, nxt);
        for (long long s = s_begin; s < s_end; ++s) {
#pragma unroll
            for (int u = 0; u < UNITS; ++u) {
                cur[u][0] = nxt[u][0];
                cur[u][1] = nxt[u][1];
            }
            const int ks_next = (ks + 1 == p.nks) ? 0 : ks + 1;
            if (s + 1 < s_end) load_stage(ks_next, nxt);
            const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(G::EMPTY_AB + stage), phase ^ 1u, abort_flag));
            if (!ok) {
                if (lane == 0) report_timeout(p.status, abort_flag, W_EMPTY_AB);
                break;
            }
            const uint32_t xt = base + (uint32_t)stage * G::STAGE_BYTES + G::W_BYTES;
#pragma unroll
            for (int u = 0; u < UNITS; ++u) {
                const int unit = qt + u * 128, m = unit >> 4, piece = unit & 15, k = ks * kBK + piece * 8;
                float f[8];
                if (wide) {
                    f[0] = __uint_as_float(cur[u][0].x); f[1] = __uint_as_float(cur[u][0].y);
                    f[2] = __uint_as_float(cur[u][0].z); f[3] = __uint_as_float(cur[u][0].w);
                    f[4] = __uint_as_float(cur[u][1].x); f[5] = __uint_as_float(cur[u][1].y);
                    f[6] = __uint_as_float(cur[u][1].z); f[7] = __uint_as_float(cur[u][1].w);
                } else {
                    const uint32_t w4[4] = {cur[u][0].x, cur[u][0].y, cur[u][0].z, cur[u][0].w};
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        if (p.x_dtype == BI8_BF16) {
                            f[2 * h] = bf16lo(w4[h]);
                            f[2 * h + 1] = bf16hi(w4[h]);
                        } else {
                            const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&w4[h]));
                            f[2 * h] = t2.x;
                            f[2 * h + 1] = t2.y;
                        }
                    }
                }
                float amax = 0.0f;
#pragma unroll
                for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
                for (int off = 1; off < LPB; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                BlockQ bq;
                bq.set(amax, !wide);
                const uint32_t lo = pack4(bq.q(f[0]), bq.q(f[1]), bq.q(f[2]), bq.q(f[3]));
                const uint32_t hi = pack4(bq.q(f[4]), bq.q(f[5]), bq.q(f[6]), bq.q(f[7]));
                if (m < p.M) {
                    // 128-byte swizzle of a K-major tile: the 16-byte chunk index is xor-ed with the row index mod 8
                    const uint32_t dst = xt + (uint32_t)(m * 128 + ((((piece >> 1) ^ (m & 7)) << 4) | ((piece & 1) << 3)));
                    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(dst), "r"(lo), "r"(hi) : "memory");
                    const int j = k / QB;
                    if ((piece % LPB) == 0 && j < p.nb) sx[j * BNS + m] = amax;
                }
            }
            fence_proxy_async_smem();            // the MMA reads the tile through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(G::FULL_AB + stage));
            if (++stage == G::STAGES) { stage = 0; phase ^= 1u; }
            ks = ks_next;
        }
    } else if (warp < PW && (warp >> 2) < p.live_chunks) {
        // ---------------- promotion + epilogue: warp = 4 * chunk + lane quarter ----------------
        const int quarter = warp & 3, chunk = warp >> 2;
        const int row = quarter * 32 + lane;                       // weight row inside the tile
        constexpr int CW = G::CW;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(chunk * CW);
        const float div = 1.0f / (127.0f * 127.0f);
        asm volatile("griddepcontrol.wait;" ::: "memory");      // activation scales, and every store, after the previous kernel

        // activation scales of all blocks, zero beyond the valid rows: [nb][BNS] (FUSED: the quantizer warps write the
        // entries of a stage before they arrive on its barrier; columns beyond M are never stored)
        const int nthreads = live_warps * 32;
        if (!FUSED) {
            const int total = p.nb * BNS;
            for (int i0 = threadIdx.x; i0 < total; i0 += nthreads * 8) {       // eight loads in flight per thread
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * nthreads, j = i / BNS, m = i % BNS;
                    v[u] = (i < total && m < p.M) ? __ldg(p.sA + (int64_t)j * p.M + m) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (i0 + u * nthreads < total) sx[i0 + u * nthreads] = v[u];
            }
            asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        }

        int stage = 0, buf = 0;
        uint32_t phase = 0, accphase = 0;
        bool ok = true;
        for (long long s = s_begin; s < s_end && ok;) {
            const int tile = (int)(s / p.nks), ks0 = (int)(s - (long long)tile * p.nks);
            const long long left = s_end - s;
            const int len = (long long)(p.nks - ks0) < left ? (p.nks - ks0) : (int)left;
            const int ks1 = ks0 + len;
            float acc[CW];
#pragma unroll
            for (int i = 0; i < CW; ++i) acc[i] = 0.0f;

            for (int ks = ks0; ks < ks1; ++ks) {
                // the stage's barrier is waited on here as well: this warp reads the scales the TMA wrote
                ok = __all_sync(0xffffffffu, mbar_wait(bar(G::FULL_AB + stage), phase, abort_flag));
                if (!ok) {
                    if (lane == 0) report_timeout(p.status, abort_flag, W_FULL_AB);
                    break;
                }
                ok = __all_sync(0xffffffffu, mbar_wait(bar(G::ACC_FULL + buf), accphase, abort_flag));
                if (!ok) {
                    if (lane == 0) report_timeout(p.status, abort_flag, W_ACC_FULL);
                    break;
                }
                tc_fence_after();
                uint32_t v[G::VB][CW];
                float sw[G::BPS];
                const uint32_t sc_u32 = base + (uint32_t)stage * G::STAGE_BYTES + G::W_BYTES + G::X_BYTES + (uint32_t)(row * 4);
#pragma unroll
                for (int b0 = 0; b0 < G::BPS; b0 += G::VB) {
#pragma unroll
                    for (int vb = 0; vb < G::VB; ++vb) {
                        const uint32_t ta = t_lane + (uint32_t)(buf * G::ACC_STRIDE + (b0 + vb) * BNS);
                        if constexpr (CW == 16) tmem_ld16(ta, v[vb]);
                        else tmem_ld32(ta, v[vb]);
                    }
                    if (b0 == 0) {
#pragma unroll
                        for (int blk = 0; blk < G::BPS; ++blk) sw[blk] = lds_f32(sc_u32 + (uint32_t)(blk * kTileRows * 4));
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(G::EMPTY_AB + stage));       // scales are in registers
                    }
                    tmem_wait_ld();
#pragma unroll
                    for (int vb = 0; vb < G::VB; ++vb) {
                        const int blk = b0 + vb, j = ks * G::BPS + blk;
                        if (j < p.nb) {
                            const uint32_t sxa = sx_u32 + (uint32_t)((j * BNS + chunk * CW) * 4);
#pragma unroll
                            for (int q = 0; q < CW / 8; ++q) {
                                uint64_t a0, a1, a2, a3;
                                lds_2xb64(sxa + (uint32_t)(q * 32), a0, a1);
                                lds_2xb64(sxa + (uint32_t)(q * 32 + 16), a2, a3);
                                float sv[8];
                                unpack_f32x2(a0, sv[0], sv[1]);
                                unpack_f32x2(a1, sv[2], sv[3]);
                                unpack_f32x2(a2, sv[4], sv[5]);
                                unpack_f32x2(a3, sv[6], sv[7]);
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    // the reference's order for one term: sB * (sA * (float(P) * 1/127^2))
                                    const float pf = __fmul_rn((float)(int32_t)v[vb][q * 8 + i], div);
                                    acc[q * 8 + i] = __fadd_rn(acc[q * 8 + i], __fmul_rn(sw[blk], __fmul_rn(sv[i], pf)));
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(G::ACC_EMPTY + buf));
                if (++stage == G::STAGES) { stage = 0; phase ^= 1u; }
                if (++buf == G::NBUF) { buf = 0; accphase ^= 1u; }
            }
            if (!ok) break;

            const int n = tile * kTileRows + row;
            if (ks0 == 0 && ks1 == p.nks) {
                if (n < p.N) {
#pragma unroll
                    for (int i = 0; i < CW; ++i) {
                        const int m = chunk * CW + i;
                        if (m < p.M) finish_store(acc[i], m, n, p.bias, p.bias_dtype, p.bias_ld, p.C, p.ldc, p.out_dtype);
                    }
                }
            } else {
                // part of a tile: slot 0 of this CTA if the part begins where the CTA's range begins, else slot 1
                const long long slot = 2ll * blockIdx.x + (s == s_begin ? 0 : 1);
                float* w = p.ws + (slot * BNS + chunk * CW) * kTileRows + row;
#pragma unroll
                for (int i = 0; i < CW; ++i)
                    if (chunk * CW + i < p.M) w[i * kTileRows] = acc[i];
            }
            s += len;
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == MW) {
        tc_fence_after();
        tmem_dealloc(tmem_base, G::TMEM_COLS);
    }
}

// Row-wise block quantizer for the few activation rows of a decode step (same arithmetic as the standalone quantizer:
// quant_math.cuh), used by the quantize-on-load entry point in front of the GEMM.  A thread takes 8 consecutive elements;
// the QB/8 lanes of a block reduce the absmax with xor shuffles.  It lets the GEMM, launched with programmatic stream
// serialisation, become resident at once: the GEMM's set-up and its first weight copies run beside this kernel and
// only its activation loads wait for it.
template <int QB>
__global__ void __launch_bounds__(256) skinny_quantize_kernel(const void* __restrict__ x, int x_dtype, int64_t ldx,
                                                              int8_t* __restrict__ q, float* __restrict__ sx, int M, int K, int nb) {
    // Launched with programmatic stream serialisation itself: resident while the kernel before it (the previous layer's
    // reduction) finishes.  Its own dependent, the GEMM, is released only after that kernel has completed, so that
    // whatever the GEMM reads early (weights, weight scales) has been at rest for a full kernel boundary.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int LPB = QB / 8;
    const int upr = nb * LPB;                                  // units per row, padded to whole blocks
    const int64_t u = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int m = (int)(u / upr), piece = (int)(u % upr), k = piece * 8;
    const bool wide = x_dtype == BI8_F32;
    const bool valid = m < M && k < K;
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = 0.0f;
    if (valid) {
        const unsigned char* src = static_cast<const unsigned char*>(x) + ((int64_t)m * ldx + k) * (wide ? 4 : 2);
        const uint4 a = ld_nc_v4(src);
        if (wide) {
            const uint4 b = ld_nc_v4(src + 16);
            f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
            f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
        } else {
            const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                if (x_dtype == BI8_BF16) {
                    f[2 * h] = bf16lo(w4[h]);
                    f[2 * h + 1] = bf16hi(w4[h]);
                } else {
                    const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&w4[h]));
                    f[2 * h] = t2.x;
                    f[2 * h + 1] = t2.y;
                }
            }
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
    for (int off = 1; off < LPB; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (!valid) return;
    BlockQ bq;
    bq.set(amax, !wide);
    const uint32_t lo = pack4(bq.q(f[0]), bq.q(f[1]), bq.q(f[2]), bq.q(f[3]));
    const uint32_t hi = pack4(bq.q(f[4]), bq.q(f[5]), bq.q(f[6]), bq.q(f[7]));
    *reinterpret_cast<uint2*>(q + (int64_t)m * K + k) = make_uint2(lo, hi);
    if ((piece % LPB) == 0) sx[(int64_t)(k / QB) * M + m] = amax;
}

// Adds the parts of divided tiles in ascending K order and writes C; tiles that one CTA covered completely were
// already written by it.  One thread per output element (a thread per tile row with a loop over the activation rows
// serialises the loads and is several times slower); `ctas` and `total_stages` are those of the GEMM launch, bns its BNS.
__global__ void __launch_bounds__(256) skinny_reduce_kernel(const float* __restrict__ ws, long long total_stages, int ctas,
                                                            int nks, int bns, const void* bias, int bias_dtype,
                                                            int64_t bias_ld, void* C, int64_t ldc, int out_dtype, int M, int N) {
    // Launched with programmatic stream serialisation: the blocks may become resident while the GEMM still runs and do
    // their index arithmetic; griddepcontrol.wait returns when the GEMM grid has completed and its stores are visible.
    // A quantizer of this library launched the same way behind this kernel (the next layer's) may become resident now.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const bool live = i < (int64_t)M * N;
    const int m = live ? (int)(i / N) : 0, n = live ? (int)(i % N) : 0;
    const int tile = n / kTileRows, row = n % kTileRows;
    const long long t0 = (long long)tile * nks, t1 = t0 + nks;
    long long c0 = t0 * ctas / total_stages;
    while (c0 + 1 < ctas && range_start(c0 + 1, total_stages, ctas) <= t0) ++c0;
    while (c0 > 0 && range_start(c0, total_stages, ctas) > t0) --c0;
    // the tile's parts belong to CTAs c0, c0 + 1, ...; a part that begins where its CTA's range begins is that CTA's
    // slot 0, and only the first part of a tile can begin elsewhere (at the tile's first stage, inside the range of c0)
    const long long cs0 = range_start(c0, total_stages, ctas);
    const bool whole = cs0 <= t0 && range_start(c0 + 1, total_stages, ctas) >= t1;   // written by the GEMM itself
    int parts = 1;
    while (range_start(c0 + parts, total_stages, ctas) < t1) ++parts;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!live || whole) return;
    float acc = __ldcg(ws + ((2 * c0 + (cs0 < t0 ? 1 : 0)) * bns + m) * kTileRows + row);
    for (int q = 1; q < parts; q += 4) {                     // four loads in flight, added in ascending order
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = (q + u < parts) ? __ldcg(ws + (2 * (c0 + q + u) * bns + m) * kTileRows + row) : 0.0f;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (q + u < parts) acc = __fadd_rn(acc, v[u]);
    }
    finish_store(acc, m, n, bias, bias_dtype, bias_ld, C, ldc, out_dtype);
}

// The same reduction for a row-parallel layer: the tile sums are this rank's partial result, and instead of writing them
// out for a second kernel the CTA exchanges them with the other ranks over peer memory right away (peer_common.cuh).  A
// thread takes four consecutive columns of a row (they lie in one tile); `part` is the fp32 [M, N] array into which the
// GEMM wrote the tiles that one CTA covered completely.  Launched for every shape, divided tiles or not.
__global__ void __launch_bounds__(kPeerThreads) skinny_reduce_peer_kernel(const float* __restrict__ ws, long long total_stages, int ctas,
                                                                          int nks, int bns, const float* __restrict__ part, int M,
                                                                          int N, const PeerArgs a, const void* bias,
                                                                          int bias_dtype, void* out, int out_dtype,
                                                                          long long limit_cycles, int* status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");       // as in skinny_reduce_kernel
    const int64_t count = (int64_t)M * N;
    const int64_t i = (int64_t)blockIdx.x * kPeerChunk + (int64_t)threadIdx.x * 4;
    const bool live = i < count;
    const int m = live ? (int)(i / N) : 0, n = live ? (int)(i % N) : 0;
    const int tile = n / kTileRows, row = n % kTileRows;
    const long long t0 = (long long)tile * nks, t1 = t0 + nks;
    long long c0 = t0 * ctas / total_stages;
    while (c0 + 1 < ctas && range_start(c0 + 1, total_stages, ctas) <= t0) ++c0;
    while (c0 > 0 && range_start(c0, total_stages, ctas) > t0) --c0;
    const long long cs0 = range_start(c0, total_stages, ctas);
    const bool whole = cs0 <= t0 && range_start(c0 + 1, total_stages, ctas) >= t1;   // written by the GEMM itself
    int parts = 1;
    while (range_start(c0 + parts, total_stages, ctas) < t1) ++parts;
    const uint32_t seq = peer_sequence(a);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        if (whole) {
            v = __ldcg(reinterpret_cast<const float4*>(part + i));
        } else {
            // parts in ascending K order, like skinny_reduce_kernel (0 + first part is exact)
            v = __ldcg(reinterpret_cast<const float4*>(ws + ((2 * c0 + (cs0 < t0 ? 1 : 0)) * bns + m) * kTileRows + row));
            for (int q = 1; q < parts; ++q) {
                const float4 w = __ldcg(reinterpret_cast<const float4*>(ws + (2 * (c0 + q) * bns + m) * kTileRows + row));
                v.x = __fadd_rn(v.x, w.x);
                v.y = __fadd_rn(v.y, w.y);
                v.z = __fadd_rn(v.z, w.z);
                v.w = __fadd_rn(v.w, w.w);
            }
        }
    }
    peer_exchange_store(a, seq, v, count, N, bias, bias_dtype, out, out_dtype, limit_cycles, status);
}

template <int QB, int BNS, bool FUSED>
int launch_skinny(const GemmArgs& g, const SkParams& p, int grid, cudaStream_t st) {
    using G = SkGeo<QB, BNS, FUSED>;
    CUtensorMap mw, mx, ms;
    int dev = 0;
    BI8_CUDA_TRY(cudaGetDevice(&dev));
    int rc = cached_operand_map(&mw, dev, g.Bt, g.N, g.K, g.ldb, kTileRows);
    if (rc != BI8_OK) return rc;
    if (FUSED) {
        mx = mw;                    // not used: the quantizer warps write the activation tile
    } else {
        rc = cached_operand_map(&mx, dev, g.A, g.M, g.K, g.lda, BNS);
        if (rc != BI8_OK) return rc;
    }
    rc = cached_scale_map(&ms, dev, g.sB, p.nb, g.N, kTileRows, G::BPS);
    if (rc != BI8_OK) return rc;
    const size_t smem = smem_of<QB, BNS, FUSED>(p.nb);
    static SmemOptIn opt_in;
    rc = opt_in.ensure(gemm_tc_skinny_kernel<QB, BNS, FUSED>, smem);
    if (rc != BI8_OK) return rc;
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(G::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;      // what may run before the predecessor has completed is decided in the kernel (early_weights)
    BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tc_skinny_kernel<QB, BNS, FUSED>, mw, mx, ms, p));
    return BI8_OK;
}

int bns_for(int64_t M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }

// dynamic shared memory of a launch; 0 for combinations that are not built
size_t skinny_smem(int block, int bns, bool fused, int nb);

size_t skinny_smem(int block, int bns, bool fused, int nb) {
#define BI8_SM(QB, BNS) \
    if (block == QB && bns == BNS) return fused ? (BNS <= 32 ? smem_of<QB, (BNS <= 32 ? BNS : 16), true>(nb) : 0) : smem_of<QB, BNS, false>(nb)
    BI8_SM(32, 16); BI8_SM(32, 32); BI8_SM(32, 64);
    BI8_SM(64, 16); BI8_SM(64, 32); BI8_SM(64, 64);
    BI8_SM(128, 16); BI8_SM(128, 32); BI8_SM(128, 64);
#undef BI8_SM
    return 0;
}

constexpr size_t kSmemLimit = 227 * 1024;

// conditions that depend on the shape only (the workspace query knows nothing else)
bool skinny_shape_ok(int64_t M, int64_t N, int64_t K, int block, bool fused = false) {
    if (M < 1 || M > kSkMaxM || N < 1 || K < 1) return false;
    if (block != 32 && block != 64 && block != 128) return false;
    if (N % 4 != 0 || N >= (1ll << 30) || K >= (1ll << 30)) return false;
    const int64_t nb = (K + block - 1) / block;
    if (nb > (1 << 20)) return false;
    const size_t smem = skinny_smem(block, bns_for(M), fused, (int)nb);
    return smem != 0 && smem <= kSmemLimit;
}

}  // namespace

// two fp32 slots of 128 x BNS per CTA
size_t gemm_skinny_workspace_bytes(const GemmArgs& g) {
    const DeviceInfo di = device_info();
    if (!di.ok || g.partials != nullptr || !skinny_shape_ok(g.M, g.N, g.K, g.block)) return 0;
    return (size_t)2 * di.sms * bns_for(g.M) * kTileRows * 4;
}

int launch_skinny_quantize(const void* x, int x_dtype, int64_t ldx, int8_t* q, float* sx, int64_t M, int64_t K, int block,
                           cudaStream_t st) {
    const int nb = (int)((K + block - 1) / block);
    const int64_t units = M * nb * (block / 8);
    const unsigned blocks = (unsigned)((units + 255) / 256);
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // the kernel waits for its predecessor itself
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    switch (block) {
        case 32: BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_quantize_kernel<32>, x, x_dtype, ldx, q, sx, (int)M, (int)K, nb)); break;
        case 64: BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_quantize_kernel<64>, x, x_dtype, ldx, q, sx, (int)M, (int)K, nb)); break;
        case 128: BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_quantize_kernel<128>, x, x_dtype, ldx, q, sx, (int)M, (int)K, nb)); break;
        default: return fail(BI8_ERR_BLOCK, "skinny quantizer supports block 32, 64, 128 (got %d)", block);
    }
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

bool gemm_skinny_applicable(const GemmArgs& g) {
    if (g.partials != nullptr || !skinny_shape_ok(g.M, g.N, g.K, g.block, g.X != nullptr)) return false;
    if (!device_info().ok) return false;
    if (!aligned(g.Bt, 16) || g.ldb % 16 != 0 || !aligned(g.sB, 16)) return false;
    if (g.X != nullptr) {
        // quantize-on-load reads 8 elements (16 or 32 bytes) at a time
        const int esz = g.x_dtype == BI8_F32 ? 4 : 2;
        if (!aligned(g.X, 16) || (g.ldx * esz) % 16 != 0 || g.K % 8 != 0) return false;
    } else if (!aligned(g.A, 16) || g.lda % 16 != 0) {
        return false;
    }
    const size_t need = gemm_skinny_workspace_bytes(g);
    return g.workspace != nullptr && g.workspace_bytes >= need && aligned(g.workspace, 16);
}

int launch_gemm_skinny(const GemmArgs& g, cudaStream_t st) {
    const DeviceInfo di = device_info();
    if (!di.ok) return fail(BI8_ERR_CUDA, "tensor-core GEMM needs a compute capability 10.x device");
    SkParams p;
    std::memset(&p, 0, sizeof(p));
    p.sA = g.sA;
    p.X = g.X;
    p.ldx = g.ldx;
    p.x_dtype = g.x_dtype;
    p.bias = g.bias;
    p.bias_ld = g.bias_ld;
    p.C = g.C;
    p.ws = static_cast<float*>(g.workspace);
    p.status = device_status_ptr();
    if (!p.status) return BI8_ERR_CUDA;
    p.ldc = g.ldc;
    p.M = (int)g.M;
    p.N = (int)g.N;
    p.K = (int)g.K;
    p.nb = (int)((g.K + g.block - 1) / g.block);
    p.nks = (int)((g.K + kBK - 1) / kBK);
    p.out_dtype = g.out_dtype;
    p.bias_dtype = g.bias_dtype;
    const int bns = bns_for(g.M), cw = bns <= 32 ? 16 : 32;
    p.live_chunks = (int)((g.M + cw - 1) / cw);
    p.early_weights = g.after_own_quantizer ? 1 : 0;
    const long long tiles = (g.N + kTileRows - 1) / kTileRows;
    p.total_stages = tiles * p.nks;
    int grid = (int)(p.total_stages < di.sms ? p.total_stages : di.sms);
    // with at least three quarters as many tiles as SMs, one whole tile per CTA (no divided tile, no reduction kernel) is
    // faster than an even split (measured: 112 tiles 14.8 against 15.7 us; 96 tiles and fewer lose)
    if (tiles <= di.sms && tiles * 4 >= (long long)di.sms * 3) grid = (int)tiles;
    const bool fused = g.X != nullptr;
    int rc = BI8_ERR_SHAPE;
#define BI8_SK(QB, BNS)                                                                                               \
    if (g.block == QB && bns == BNS) {                                                                                \
        if (fused) rc = launch_skinny<QB, (BNS <= 32 ? BNS : 16), true>(g, p, grid, st);                              \
        else rc = launch_skinny<QB, BNS, false>(g, p, grid, st);                                                      \
    }
    BI8_SK(32, 16) BI8_SK(32, 32) BI8_SK(32, 64)
    BI8_SK(64, 16) BI8_SK(64, 32) BI8_SK(64, 64)
    BI8_SK(128, 16) BI8_SK(128, 32) BI8_SK(128, 64)
#undef BI8_SK
    if (rc != BI8_OK) return rc;
    if (g.peer != nullptr) {
        // row-parallel layer: the reduction kernel also exchanges the sums with the other ranks and writes the layer's output
        const PeerEpilogue& pe = *g.peer;
        const int64_t count = g.M * g.N;
        cudaLaunchConfig_t pc;
        std::memset(&pc, 0, sizeof(pc));
        pc.gridDim = dim3((unsigned)((count + kPeerChunk - 1) / kPeerChunk));
        pc.blockDim = dim3(kPeerThreads);
        pc.stream = st;
        cudaLaunchAttribute pa[1];
        pa[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see skinny_reduce_kernel
        pa[0].val.programmaticStreamSerializationAllowed = 1;
        pc.attrs = pa;
        pc.numAttrs = 1;
        BI8_CUDA_TRY(cudaLaunchKernelEx(&pc, skinny_reduce_peer_kernel, (const float*)p.ws, p.total_stages, grid, p.nks, bns,
                                        (const float*)g.C, (int)g.M, (int)g.N, *static_cast<const PeerArgs*>(pe.args), pe.bias,
                                        pe.bias_dtype, pe.out, pe.out_dtype, pe.limit_cycles, p.status));
        return BI8_OK;
    }
    if (p.total_stages % grid == 0 && (p.total_stages / grid) % p.nks == 0) return BI8_OK;   // no tile is divided
    const int64_t total = g.M * g.N;
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)((total + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see skinny_reduce_kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BI8_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_reduce_kernel, (const float*)p.ws, p.total_stages, grid, p.nks, bns,
                                    g.bias, g.bias_dtype, g.bias_ld, g.C, g.ldc, g.out_dtype, (int)g.M, (int)g.N));
    return BI8_OK;
}

}  // namespace bi8
