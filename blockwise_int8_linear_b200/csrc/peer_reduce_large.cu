// Sum of the ranks' fp32 partial results of a row-parallel layer for prefill-sized batches: reduce-scatter by peer loads,
// all-gather by peer stores, one kernel per rank.
//
// The exchange of peer_reduce.cu pushes every rank's whole partial result to every rank (world x the bytes), which is
// right for the 128 KB of a decode step and wrong for the 64 MB of a prefill step.  Here every rank owns one chunk in
// `world` of the result (chunk c belongs to rank c mod world).  The ranks' partial results already lie in peer-mapped
// memory: the GEMM wrote them there.  A rank
//   1. announces that its partial result is complete (flag `ready` on every rank; the GEMM ran earlier in its stream),
//   2. waits, bounded, for the other ranks' announcements,
//   3. for each of its chunks loads the chunk from every rank's partial result (plain 16-byte loads from peer addresses),
//      adds them in ascending rank order, casts, adds bias or residual in the output type and stores the chunk into EVERY
//      rank's output region (plain stores to peer addresses),
//   4. when all its CTAs are through, sets flag `done` on every rank, and its last CTA waits, bounded, for the other
//      ranks' `done` flags before the kernel ends: whatever follows in the stream finds the complete output.
// Per rank (world - 1) / world of the fp32 result comes in over NVLink and (world - 1) / world of the cast result goes
// out, against twice the fp32 result each way for a ring all-reduce.  A rank leaves the kernel only when every rank has
// finished reading its partial result and writing into its output, and it enters the next one only after the consumers of
// this output have run, so one partial region, one output region and two flag rows per rank suffice; the flags carry a
// sequence number that lives in device memory (the launch can be captured and replayed).  Peer memory is touched by
// nothing but these loads and stores.  The sum is bit-identical on all ranks (one rank computes each element) and equal
// to peer_reduce.cu's (same order).
#include "peer_common.cuh"

namespace bi8 {
namespace {

constexpr size_t kLargeCtrlBytes = 1024;          // sequence pair, ready[8], done[8]
enum { PW_READY = 2, PW_DONE = 3 };

struct LargeArgs {
    unsigned char* base[kMaxRanks];               // rank r's buffer as mapped on this device
    int rank, world;
    int64_t capacity;                             // fp32 values of the partial region
};

__device__ __forceinline__ uint32_t* ctrl_seq(unsigned char* b) { return reinterpret_cast<uint32_t*>(b); }
__device__ __forceinline__ uint32_t* ctrl_ready(unsigned char* b) { return reinterpret_cast<uint32_t*>(b + 64); }
__device__ __forceinline__ uint32_t* ctrl_done(unsigned char* b) { return reinterpret_cast<uint32_t*>(b + 128); }

// waits until flags[0 .. world) all equal seq; threads 0 .. world-1 of the CTA poll one flag each.  Returns false (to all
// threads of the CTA) when the limit ran out.
__device__ __forceinline__ bool wait_flags(const uint32_t* flags, int world, uint32_t seq, long long limit_cycles, int* status, int code,
                                           int* ok_flag) {
    const int tid = threadIdx.x;
    if (tid == 0) *ok_flag = 1;
    __syncthreads();
    if (tid < world) {
        const long long t0 = clock64();
        while (ld_acquire_sys(flags + tid) != seq) {
            if (clock64() - t0 > limit_cycles) {
                *ok_flag = 0;
                if (atomicCAS(status, 0, BI8_ERR_TIMEOUT) == 0) status[1] = code;
                break;
            }
            __nanosleep(128);
        }
    }
    __syncthreads();
    return *ok_flag != 0;
}

// W: compile-time bound on the number of ranks (2, 4 or 8); U = 8 / W chunks per loop iteration, so that a thread has eight
// 16-byte loads in flight whatever the group size (the loads cross NVLink: a few microseconds each).
template <int W, int U>
__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_large_kernel(const LargeArgs a, int64_t count, int64_t n_cols,
                                                                            const void* bias, int bias_dtype, int out_dtype,
                                                                            long long limit_cycles, int* status) {
    __shared__ int ok_flag;
    __shared__ int last_flag;
    const int tid = threadIdx.x;
    unsigned char* mine = a.base[a.rank];
    const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(ctrl_seq(mine)) + 1u;
    const size_t out_off = kLargeCtrlBytes + (size_t)a.capacity * 4;

    // 1. this rank's partial result was complete before the kernel started
    if (blockIdx.x == 0 && tid < a.world) st_release_sys(ctrl_ready(a.base[tid]) + a.rank, seq);
    // 2. everybody else's
    bool ok = wait_flags(ctrl_ready(mine), a.world, seq, limit_cycles, status, PW_READY, &ok_flag);

    // 3. this rank's chunks: chunk c belongs to rank c mod world
    if (ok) {
        const int64_t chunks = (count + kPeerChunk - 1) / kPeerChunk;
        const bool full = (bias_dtype & BI8_ADDEND_FULL) != 0;
        const int bdt = bias_dtype & ~BI8_ADDEND_FULL;
        const bool hb = bias != nullptr;
        for (int64_t k0 = (int64_t)blockIdx.x; ; k0 += (int64_t)gridDim.x * U) {
            if (a.rank + a.world * k0 >= chunks) break;
            float4 p[U][W];
            int64_t i0[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t c = a.rank + a.world * (k0 + (int64_t)u * gridDim.x);
                i0[u] = c < chunks ? c * kPeerChunk + (int64_t)tid * 4 : count;
#pragma unroll
                for (int r = 0; r < W; ++r)
                    if (r < a.world && i0[u] < count) p[u][r] = ld_volatile_f4(reinterpret_cast<const float*>(a.base[r] + kLargeCtrlBytes) + i0[u]);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (i0[u] >= count) continue;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int r = 0; r < W; ++r) {
                    if (r < a.world) {
                        acc.x = __fadd_rn(acc.x, p[u][r].x);
                        acc.y = __fadd_rn(acc.y, p[u][r].y);
                        acc.z = __fadd_rn(acc.z, p[u][r].z);
                        acc.w = __fadd_rn(acc.w, p[u][r].w);
                    }
                }
                float s[4] = {acc.x, acc.y, acc.z, acc.w};
                float b[4] = {0.f, 0.f, 0.f, 0.f};
                if (hb) {
                    const int64_t col = full ? i0[u] : i0[u] % n_cols;    // n_cols is a multiple of 4: the four values share a row
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (bdt == BI8_BF16) b[e] = __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[col + e]);
                        else if (bdt == BI8_F16) b[e] = __half2float(static_cast<const __half*>(bias)[col + e]);
                        else b[e] = static_cast<const float*>(bias)[col + e];
                    }
                }
                if (out_dtype == BI8_F32) {
                    const float4 o = make_float4(hb ? __fadd_rn(s[0], b[0]) : s[0], hb ? __fadd_rn(s[1], b[1]) : s[1],
                                                 hb ? __fadd_rn(s[2], b[2]) : s[2], hb ? __fadd_rn(s[3], b[3]) : s[3]);
#pragma unroll
                    for (int r = 0; r < W; ++r)
                        if (r < a.world) *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.base[r] + out_off) + i0[u]) = o;
                } else {
                    uint2 o;
                    if (out_dtype == BI8_BF16) {
                        __nv_bfloat16 h[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            h[e] = __float2bfloat16_rn(s[e]);
                            // the addend comes after the cast, in the output type, as in the unsharded layer
                            if (hb) h[e] = __float2bfloat16_rn(__fadd_rn(__bfloat162float(h[e]), __bfloat162float(__float2bfloat16_rn(b[e]))));
                        }
                        o = *reinterpret_cast<uint2*>(h);
                    } else {
                        __half h[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            h[e] = __float2half_rn(s[e]);
                            if (hb) h[e] = __float2half_rn(__fadd_rn(__half2float(h[e]), __half2float(__float2half_rn(b[e]))));
                        }
                        o = *reinterpret_cast<uint2*>(h);
                    }
#pragma unroll
                    for (int r = 0; r < W; ++r)
                        if (r < a.world) *reinterpret_cast<uint2*>(a.base[r] + out_off + (size_t)i0[u] * 2) = o;
                }
            }
        }
    }

    // 4. the rank's last CTA tells everybody and waits for everybody
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const uint32_t done = atomicAdd(ctrl_seq(mine) + 1, 1u) + 1u;
        last_flag = done == gridDim.x;
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence_system();
    if (tid < a.world) st_release_sys(ctrl_done(a.base[tid]) + a.rank, seq);
    wait_flags(ctrl_done(mine), a.world, seq, limit_cycles, status, PW_DONE, &ok_flag);
    if (tid == 0) {
        ctrl_seq(mine)[1] = 0u;
        __threadfence();
        ctrl_seq(mine)[0] = seq;           // the next launch (or replay) continues the sequence
    }
}

}  // namespace

size_t peer_allreduce_large_buffer_bytes(int64_t capacity) {
    // control block, the partial region (fp32), the output region (room for fp32 output)
    return kLargeCtrlBytes + (size_t)capacity * 4 + (size_t)capacity * 4;
}

size_t peer_allreduce_large_partial_offset() { return kLargeCtrlBytes; }
size_t peer_allreduce_large_out_offset(int64_t capacity) { return kLargeCtrlBytes + (size_t)capacity * 4; }

int launch_peer_allreduce_large(void* const* peer_bufs, int rank, int world, int64_t capacity, int64_t M, int64_t N, const void* bias,
                                int bias_dtype, int out_dtype, unsigned wait_limit_us, cudaStream_t st) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return fail(BI8_ERR_SHAPE, "peer all-reduce: rank %d of %d", rank, world);
    if (capacity <= 0 || capacity % kPeerChunk != 0) return fail(BI8_ERR_SHAPE, "peer all-reduce: capacity must be a positive multiple of %d", kPeerChunk);
    const int64_t count = M * N;
    if (M <= 0 || N <= 0 || N % 4 != 0 || count > capacity)
        return fail(BI8_ERR_SHAPE, "peer all-reduce: M*N = %lld does not fit the buffers (capacity %lld, N a multiple of 4)", (long long)count, (long long)capacity);
    LargeArgs a;
    for (int r = 0; r < kMaxRanks; ++r) {
        unsigned char* base = static_cast<unsigned char*>(peer_bufs[r < world ? r : 0]);
        if (!base || !aligned(base, 16)) return fail(BI8_ERR_NULL, "peer all-reduce: buffer of rank %d", r);
        a.base[r] = base;
    }
    a.rank = rank;
    a.world = world;
    a.capacity = capacity;
    int* status = device_status_ptr();
    if (!status) return BI8_ERR_CUDA;
    int dev = 0, sms = 0;
    BI8_CUDA_TRY(cudaGetDevice(&dev));
    BI8_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t my_chunks = ((count + kPeerChunk - 1) / kPeerChunk + world - 1) / world;
    const long long limit = peer_wait_limit_cycles(wait_limit_us);
#define BI8_LARGE(W, U)                                                                                                          \
    do {                                                                                                                         \
        int per_sm = 0;                                                                                                          \
        BI8_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, peer_allreduce_large_kernel<W, U>, kPeerThreads, 0)); \
        const int64_t want = (my_chunks + U - 1) / U, room = (int64_t)sms * (per_sm > 0 ? per_sm : 1);                            \
        const unsigned grid = (unsigned)(want < 1 ? 1 : (want < room ? want : room));                                            \
        peer_allreduce_large_kernel<W, U><<<grid, kPeerThreads, 0, st>>>(a, count, N, bias, bias_dtype, out_dtype, limit, status); \
    } while (0)
    if (world <= 2) BI8_LARGE(2, 4);
    else if (world <= 4) BI8_LARGE(4, 2);
    else BI8_LARGE(8, 1);
#undef BI8_LARGE
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

}  // namespace bi8
