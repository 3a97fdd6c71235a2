// Sum of the ranks' fp32 partial results of a row-parallel layer over NVLink peer memory, one kernel per rank.
//
// A row-parallel BlockInt8Linear (the K dimension of block_linear.py:141-143 divided over ranks on block boundaries)
// leaves an fp32 partial result [M, N] on every rank; the layer's output is their sum in rank order, cast, plus bias.
// For decode-sized M the NCCL all-reduce of those 128 KB costs 10-60 us of launch and protocol latency per layer and has
// to stay outside a CUDA graph that is replayed by every rank on its own; this kernel does the exchange with plain
// stores and loads on peer-mapped memory and can be captured like any other kernel:
//   1. every CTA takes one chunk of the data, writes its rank's values of that chunk into slot [rank] of EVERY rank's
//      receive buffer (st.global to peer addresses; its own buffer included), fences at system scope, and sets the chunk's
//      flag [rank] on every rank to the current sequence number (st.release.sys);
//   2. it waits until the chunk's flags of all ranks in ITS OWN buffer carry that sequence number (ld.acquire.sys, bounded:
//      when the limit runs out it records BI8_ERR_TIMEOUT in the status word and returns without touching the output);
//   3. it adds the world's slots of the chunk in ascending rank order (the same order on every rank: all ranks end with
//      bit-identical results), casts, adds bias in the output type and stores.
// Receive buffers and flags alternate between two sets by sequence parity: a rank can be at most one reduction ahead of
// the slowest one (it needs that rank's flags to finish), so a set is never overwritten while a peer still reads it.
// The sequence number lives in device memory and is advanced by the last CTA to finish, so that replays of a captured
// launch continue the sequence.
//
// The peer buffers are only ever touched by this kernel's plain loads and stores: no tensor map, no bulk copy, no
// multicast object, no library kernel sees them.
#include "bi8_common.cuh"

namespace bi8 {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kChunk = 1024;          // fp32 values per CTA: 256 threads x 4
constexpr int kPeerThreads = 256;
enum { PW_FLAGS = 1 };

struct PeerArgs {
    float* slots[kMaxRanks];          // rank r's receive buffer: [2 sets][world][capacity] fp32
    uint32_t* flags[kMaxRanks];       // rank r's flags: [2 sets][world][capacity / kChunk] u32
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

__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_kernel(const PeerArgs a, const float* __restrict__ partial,
                                                                      int64_t count, int64_t n_cols, const void* __restrict__ bias,
                                                                      int bias_dtype, void* __restrict__ out, int out_dtype,
                                                                      long long limit_cycles, int* status) {
    __shared__ int ok_flag;
    const int tid = threadIdx.x;
    const int64_t chunk = blockIdx.x;
    const int64_t chunks_cap = a.capacity / kChunk;
    const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(a.seq) + 1u;      // this reduction's number (never 0)
    const int set = (int)(seq & 1u);
    const int64_t i0 = chunk * kChunk + (int64_t)tid * 4;
    if (tid == 0) ok_flag = 1;

    // 1. this rank's values of the chunk into every rank's slot [rank]
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i0 < count) v = *reinterpret_cast<const float4*>(partial + i0);
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

    // 2. wait for every rank's flag of this chunk in this rank's own buffer
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

    // 3. sum in rank order, cast, bias, store
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
        const int64_t col = i0 % n_cols;              // n_cols is a multiple of 4: the four values share a row
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

}  // namespace

size_t peer_allreduce_buffer_bytes(int world, int64_t capacity) {
    // [2][world][capacity] fp32 slots, then [2][world][capacity / kChunk] u32 flags, then the sequence counter pair
    const int64_t chunks = capacity / kChunk;
    return (size_t)(2 * world * capacity * 4 + 2 * world * chunks * 4 + 16);
}

int launch_peer_allreduce(void* const* peer_bufs, int rank, int world, int64_t capacity, const float* partial, int64_t M, int64_t N,
                          const void* bias, int bias_dtype, void* out, int out_dtype, unsigned wait_limit_us, cudaStream_t st) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return fail(BI8_ERR_SHAPE, "peer all-reduce: rank %d of %d", rank, world);
    if (capacity <= 0 || capacity % kChunk != 0) return fail(BI8_ERR_SHAPE, "peer all-reduce: capacity must be a positive multiple of %d", kChunk);
    const int64_t count = M * N;
    if (M <= 0 || N <= 0 || N % 4 != 0 || count > capacity) return fail(BI8_ERR_SHAPE, "peer all-reduce: M*N = %lld does not fit the buffers (capacity %lld, N a multiple of 4)", (long long)count, (long long)capacity);
    if (!aligned(partial, 16) || !aligned(out, 16)) return fail(BI8_ERR_ALIGN, "peer all-reduce: partial and out must be 16-byte aligned");
    PeerArgs a;
    const int64_t chunks = capacity / kChunk;
    for (int r = 0; r < kMaxRanks; ++r) {
        unsigned char* base = static_cast<unsigned char*>(peer_bufs[r < world ? r : 0]);
        if (!base || !aligned(base, 16)) return fail(BI8_ERR_NULL, "peer all-reduce: buffer of rank %d", r);
        a.slots[r] = reinterpret_cast<float*>(base);
        a.flags[r] = reinterpret_cast<uint32_t*>(base + (size_t)2 * world * capacity * 4);
    }
    a.seq = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(peer_bufs[rank]) + (size_t)2 * world * capacity * 4 + (size_t)2 * world * chunks * 4);
    a.rank = rank;
    a.world = world;
    a.capacity = capacity;
    int* status = device_status_ptr();
    if (!status) return BI8_ERR_CUDA;
    // SM clock of at most ~2 GHz: the limit in cycles errs on the long side
    const long long limit = (long long)(wait_limit_us ? wait_limit_us : 1000000u) * 2000ll;
    const unsigned grid = (unsigned)((count + kChunk - 1) / kChunk);
    peer_allreduce_kernel<<<grid, kPeerThreads, 0, st>>>(a, partial, count, N, bias, bias_dtype, out, out_dtype, limit, status);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

}  // namespace bi8
