// Sum of the ranks' fp32 partial results of a row-parallel layer over NVLink peer memory, one kernel per rank.
//
// A row-parallel BlockInt8Linear (the K dimension of block_linear.py:141-143 divided over ranks on block boundaries)
// leaves an fp32 partial result [M, N] on every rank; the layer's output is their sum in rank order, cast, plus bias.
// For decode-sized M the NCCL all-reduce of those 128 KB costs 10-60 us of launch and protocol latency per layer and has
// to stay outside a CUDA graph that is replayed by every rank on its own; this kernel does the exchange with plain
// stores and loads on peer-mapped memory and can be captured like any other kernel.  This file holds the stand-alone
// kernel and the host side; the protocol itself is in peer_common.cuh, and the decode GEMM's reduction kernel runs it
// on the tile sums it has just formed (gemm_tc_skinny.cu).
#include "peer_common.cuh"

namespace bi8 {
namespace {

__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_kernel(const PeerArgs a, const float* __restrict__ partial,
                                                                      int64_t count, int64_t n_cols, const void* bias,
                                                                      int bias_dtype, void* out, int out_dtype,
                                                                      long long limit_cycles, int* status) {
    const uint32_t seq = peer_sequence(a);
    const int64_t i0 = (int64_t)blockIdx.x * kPeerChunk + (int64_t)threadIdx.x * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i0 < count) v = *reinterpret_cast<const float4*>(partial + i0);
    peer_exchange_store(a, seq, v, count, n_cols, bias, bias_dtype, out, out_dtype, limit_cycles, status);
}

}  // namespace

size_t peer_allreduce_buffer_bytes(int world, int64_t capacity) {
    // [2][world][capacity] fp32 slots, then [2][world][capacity / kPeerChunk] u32 flags, then the sequence counter pair
    const int64_t chunks = capacity / kPeerChunk;
    return (size_t)(2 * world * capacity * 4 + 2 * world * chunks * 4 + 16);
}

int make_peer_args(PeerArgs* a, void* const* peer_bufs, int rank, int world, int64_t capacity, int64_t M, int64_t N) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return fail(BI8_ERR_SHAPE, "peer all-reduce: rank %d of %d", rank, world);
    if (capacity <= 0 || capacity % kPeerChunk != 0) return fail(BI8_ERR_SHAPE, "peer all-reduce: capacity must be a positive multiple of %d", kPeerChunk);
    const int64_t count = M * N;
    if (M <= 0 || N <= 0 || N % 4 != 0 || count > capacity) return fail(BI8_ERR_SHAPE, "peer all-reduce: M*N = %lld does not fit the buffers (capacity %lld, N a multiple of 4)", (long long)count, (long long)capacity);
    const int64_t chunks = capacity / kPeerChunk;
    for (int r = 0; r < kMaxRanks; ++r) {
        unsigned char* base = static_cast<unsigned char*>(peer_bufs[r < world ? r : 0]);
        if (!base || !aligned(base, 16)) return fail(BI8_ERR_NULL, "peer all-reduce: buffer of rank %d", r);
        a->slots[r] = reinterpret_cast<float*>(base);
        a->flags[r] = reinterpret_cast<uint32_t*>(base + (size_t)2 * world * capacity * 4);
    }
    a->seq = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(peer_bufs[rank]) + (size_t)2 * world * capacity * 4 + (size_t)2 * world * chunks * 4);
    a->rank = rank;
    a->world = world;
    a->capacity = capacity;
    return BI8_OK;
}

// SM clock of at most ~2 GHz: the limit in cycles errs on the long side
long long peer_wait_limit_cycles(unsigned wait_limit_us) { return (long long)(wait_limit_us ? wait_limit_us : 1000000u) * 2000ll; }

int launch_peer_allreduce(void* const* peer_bufs, int rank, int world, int64_t capacity, const float* partial, int64_t M, int64_t N,
                          const void* bias, int bias_dtype, void* out, int out_dtype, unsigned wait_limit_us, cudaStream_t st) {
    PeerArgs a;
    const int rc = make_peer_args(&a, peer_bufs, rank, world, capacity, M, N);
    if (rc != BI8_OK) return rc;
    if (!aligned(partial, 16) || !aligned(out, 16)) return fail(BI8_ERR_ALIGN, "peer all-reduce: partial and out must be 16-byte aligned");
    int* status = device_status_ptr();
    if (!status) return BI8_ERR_CUDA;
    const int64_t count = M * N;
    const unsigned grid = (unsigned)((count + kPeerChunk - 1) / kPeerChunk);
    peer_allreduce_kernel<<<grid, kPeerThreads, 0, st>>>(a, partial, count, N, bias, bias_dtype, out, out_dtype,
                                                         peer_wait_limit_cycles(wait_limit_us), status);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

}  // namespace bi8
