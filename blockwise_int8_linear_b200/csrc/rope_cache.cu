// One decode step's rotary embedding and cache append for a Llama-style attention layer, in one kernel.
//
// Not part of the reference (which has no model code of its own): between the q/k/v projection and the attention call of a
// decode step a model rotates q and k by the position's angle and appends k and v to the cache.  Written with tensor
// operations that is a conversion to fp32, a complex multiply, a conversion back and two indexed copies: five launches of
// a few microseconds each per layer, between two of this library's kernels.  Here one thread takes one (even, odd) feature
// pair of one head: q and k are rotated in fp32 ((x0 + i x1) * (c + i s), every product and sum rounded on its own) and
// rounded to the activation type, q goes to its output, k and v go to row `pos` of the caches.  `pos` is read from
// device memory, so the launch can be captured in a CUDA graph and replayed while the position advances.
#include "bi8_common.cuh"

namespace bi8 {
namespace {

template <typename T>
__device__ __forceinline__ float2 load_pair(const T* p);
template <>
__device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <>
__device__ __forceinline__ float2 load_pair<__half>(const __half* p) {
    return __half22float2(*reinterpret_cast<const __half2*>(p));
}
template <typename T>
__device__ __forceinline__ void store_pair(T* p, float a, float b);
template <>
__device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
template <>
__device__ __forceinline__ void store_pair<__half>(__half* p, float a, float b) {
    *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b);
}

// qkv [B, 3, H, D]; cis [D/2] (cos, sin) of this step's position; q_out [B, H, D]; caches [B, H, max_len, D]
template <typename T>
__global__ void __launch_bounds__(256) rope_cache_append_kernel(const T* __restrict__ qkv, const float2* __restrict__ cis,
                                                                const long long* __restrict__ pos, T* __restrict__ q_out,
                                                                T* __restrict__ kcache, T* __restrict__ vcache, int B, int H, int D,
                                                                int max_len) {
    const int half = D / 2;
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (int64_t)B * H * half) return;
    const long long p = *pos;
    if (p < 0 || p >= max_len) return;                    // a position outside the cache: nothing is written
    const int pair = (int)(i % half), h = (int)((i / half) % H), b = (int)(i / ((int64_t)half * H));
    const int64_t in = (((int64_t)b * 3) * H + h) * D + 2 * pair;
    const int64_t plane = (int64_t)H * D;
    const float2 cs = cis[pair];
    const float2 q = load_pair(qkv + in), k = load_pair(qkv + in + plane), v = load_pair(qkv + in + 2 * plane);
    const float qr = __fsub_rn(__fmul_rn(q.x, cs.x), __fmul_rn(q.y, cs.y)), qi = __fadd_rn(__fmul_rn(q.x, cs.y), __fmul_rn(q.y, cs.x));
    const float kr = __fsub_rn(__fmul_rn(k.x, cs.x), __fmul_rn(k.y, cs.y)), ki = __fadd_rn(__fmul_rn(k.x, cs.y), __fmul_rn(k.y, cs.x));
    store_pair(q_out + ((int64_t)b * H + h) * D + 2 * pair, qr, qi);
    const int64_t c = (((int64_t)b * H + h) * max_len + p) * D + 2 * pair;
    store_pair(kcache + c, kr, ki);
    store_pair(vcache + c, v.x, v.y);
}

}  // namespace

int launch_rope_cache_append(const void* qkv, int dt, const float* cis, const long long* pos, void* q_out, void* kcache, void* vcache,
                             int64_t B, int64_t H, int64_t D, int64_t max_len, cudaStream_t st) {
    const int64_t n = B * H * (D / 2);
    if (n == 0) return BI8_OK;
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (dt == BI8_BF16)
        rope_cache_append_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(qkv), reinterpret_cast<const float2*>(cis), pos, static_cast<__nv_bfloat16*>(q_out),
            static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache), (int)B, (int)H, (int)D, (int)max_len);
    else
        rope_cache_append_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(qkv), reinterpret_cast<const float2*>(cis), pos,
                                                              static_cast<__half*>(q_out), static_cast<__half*>(kcache),
                                                              static_cast<__half*>(vcache), (int)B, (int)H, (int)D, (int)max_len);
    BI8_CUDA_TRY(cudaGetLastError());
    return BI8_OK;
}

}  // namespace bi8
