// Device side of the peer-memory reduction, shared by the stand-alone kernel (peer_reduce.cu) and by the reduction kernel
// of the decode GEMM, which exchanges the tile sums it has just formed (gemm_tc_skinny.cu).
//
// Protocol for one chunk of kPeerChunk fp32 values, run by one CTA of kPeerThreads threads (four values per thread):
//   1. the rank's values go into slot [rank] of EVERY rank's receive buffer (plain 16-byte stores to peer addresses), then a
//      system-scope fence, then the chunk's flag [rank] on every rank is set to the sequence number (st.release.sys);
//   2. the CTA waits until the chunk's flags of all ranks in ITS OWN buffer carry that number (ld.acquire.sys; bounded: when
//      the limit runs out it records BI8_ERR_TIMEOUT in the status word and the chunk's output is left untouched);
//   3. it adds the world's slots of the chunk in ascending rank order (bit-identical on all ranks), casts, adds bias in the
//      output type and stores.
// Receive buffers and flags alternate between two sets by sequence parity: a rank can be at most one reduction ahead of the
// slowest one (it needs that rank's flags to finish), so a set is never overwritten while a peer still reads it.  The
// sequence number lives in device memory and is advanced by the last CTA to finish, so replays of a captured launch continue
// the sequence.  Peer memory is only touched by these plain loads and stores.
#pragma once

#include "bi8_common.cuh"

namespace bi8 {

constexpr int kMaxRanks = 8;
constexpr int kPeerChunk = 1024;      // fp32 values per CTA: 256 threads x 4
constexpr int kPeerThreads = 256;
enum { PW_FLAGS = 1 };

struct PeerArgs {
    float* slots[kMaxRanks];          // rank r's receive buffer: [2 sets][world][capacity] fp32
    uint32_t* flags[kMaxRanks];       // rank r's flags: [2 sets][world][capacity / kPeerChunk] u32
    uint32_t* seq;                    // this rank's sequence counter {value, CTAs finished}
    int rank, world;
    int64_t capacity;                 // fp32 values per slot
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// values another GPU wrote into this GPU's memory: never from L1
__device__ __forceinline__ float4 ld_volatile_f4(const float* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// This reduction's sequence number (never 0), read by every thread at the start of the kernel.
__device__ __forceinline__ uint32_t peer_sequence(const PeerArgs& a) { return *reinterpret_cast<volatile uint32_t*>(a.seq) + 1u; }

// Steps 1-3 for the chunk blockIdx.x: `v` are this thread's four values (elements i0 .. i0+3 of the flattened [M, n_cols]
// result, i0 = chunk * kPeerChunk + 4 * threadIdx.x; ignored where i0 >= count).  Must be called by all threads of the CTA.
__device__ __forceinline__ void peer_exchange_store(const PeerArgs& a, uint32_t seq, float4 v, int64_t count, int64_t n_cols,
                                                    const void* bias, int bias_dtype, void* out,
                                                    int out_dtype, long long limit_cycles, int* status) {
    __shared__ int ok_flag;
    const int tid = threadIdx.x;
    const int64_t chunk = blockIdx.x;
    const int64_t chunks_cap = a.capacity / kPeerChunk;
    const int set = (int)(seq & 1u);
    const int64_t i0 = chunk * kPeerChunk + (int64_t)tid * 4;
    if (tid == 0) ok_flag = 1;

    const int64_t slot_off = ((int64_t)set * a.world + a.rank) * a.capacity + i0;
    if (i0 < count) {
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < a.world) *reinterpret_cast<float4*>(a.slots[r] + slot_off) = v;
    }
    __threadfence_system();
    __syncthreads();
    const int64_t flag_off = ((int64_t)set * a.world) * chunks_cap + chunk;
    if (tid < a.world) st_release_sys(a.flags[tid] + flag_off + (int64_t)a.rank * chunks_cap, seq);

    if (tid < a.world) {
        const uint32_t* f = a.flags[a.rank] + flag_off + (int64_t)tid * chunks_cap;
        const long long t0 = clock64();
        bool ok = true;
        while (ld_acquire_sys(f) != seq) {
            if (clock64() - t0 > limit_cycles) {
                ok = false;
                break;
            }
            __nanosleep(64);
        }
        if (!ok) {
            ok_flag = 0;
            if (atomicCAS(status, 0, BI8_ERR_TIMEOUT) == 0) status[1] = PW_FLAGS;
        }
    }
    __syncthreads();

    if (ok_flag && i0 < count) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* mine = a.slots[a.rank] + ((int64_t)set * a.world) * a.capacity + i0;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            if (r < a.world) {
                const float4 p = ld_volatile_f4(mine + (int64_t)r * a.capacity);
                acc.x = __fadd_rn(acc.x, p.x);
                acc.y = __fadd_rn(acc.y, p.y);
                acc.z = __fadd_rn(acc.z, p.z);
                acc.w = __fadd_rn(acc.w, p.w);
            }
        }
        float s[4] = {acc.x, acc.y, acc.z, acc.w};
        // n_cols is a multiple of 4: the four values share a row.  A bias has one value per column; with BI8_ADDEND_FULL in
        // its type code the operand is a contiguous [M, n_cols] addend (a residual) indexed like the result.
        const bool full = (bias_dtype & BI8_ADDEND_FULL) != 0;
        bias_dtype &= ~BI8_ADDEND_FULL;
        const int64_t col = full ? i0 : i0 % n_cols;
        float b[4] = {0.f, 0.f, 0.f, 0.f};
        const bool hb = bias != nullptr;
        if (hb) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (bias_dtype == BI8_BF16) b[u] = __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[col + u]);
                else if (bias_dtype == BI8_F16) b[u] = __half2float(static_cast<const __half*>(bias)[col + u]);
                else b[u] = static_cast<const float*>(bias)[col + u];
            }
        }
        if (out_dtype == BI8_F32) {
            float4 o = make_float4(hb ? __fadd_rn(s[0], b[0]) : s[0], hb ? __fadd_rn(s[1], b[1]) : s[1],
                                   hb ? __fadd_rn(s[2], b[2]) : s[2], hb ? __fadd_rn(s[3], b[3]) : s[3]);
            *reinterpret_cast<float4*>(static_cast<float*>(out) + i0) = o;
        } else if (out_dtype == BI8_BF16) {
            __nv_bfloat16 o[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                o[u] = __float2bfloat16_rn(s[u]);
                // the bias is added after the cast, in the output type, as in the unsharded layer
                if (hb) o[u] = __float2bfloat16_rn(__fadd_rn(__bfloat162float(o[u]), __bfloat162float(__float2bfloat16_rn(b[u]))));
            }
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + i0) = *reinterpret_cast<uint2*>(o);
        } else {
            __half o[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                o[u] = __float2half_rn(s[u]);
                if (hb) o[u] = __float2half_rn(__fadd_rn(__half2float(o[u]), __half2float(__float2half_rn(b[u]))));
            }
            *reinterpret_cast<uint2*>(static_cast<__half*>(out) + i0) = *reinterpret_cast<uint2*>(o);
        }
    }

    // the last CTA to finish advances the sequence number for the next launch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const uint32_t done = atomicAdd(a.seq + 1, 1u) + 1u;
        if (done == gridDim.x) {
            a.seq[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(a.seq) = seq;
        }
    }
}

// Host side (peer_reduce.cu): fills PeerArgs from the ranks' buffer addresses after checking the geometry.
int make_peer_args(PeerArgs* a, void* const* peer_bufs, int rank, int world, int64_t capacity, int64_t M, int64_t N);
long long peer_wait_limit_cycles(unsigned wait_limit_us);

}  // namespace bi8
