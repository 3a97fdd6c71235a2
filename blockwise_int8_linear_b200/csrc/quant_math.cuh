// The arithmetic of one quantisation block (reference kernel triton_functions.py:397-403), shared by the standalone
// quantizers and by the GEMM that quantizes its activations on load.
#pragma once

#include "bi8_common.cuh"

namespace bi8 {

constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to integer (RNE) in the low mantissa bits

// Quantizer of one block: scale and the reciprocal used by the exact-division shortcut.
//
// For operands with at most 11 significant bits (bf16, fp16) the correctly rounded fp32 quotient a/b is
//   q0 = a*r;  e = fma(-b, q0, a);  q1 = fma(e, r, q0)        with r = RN(1/b):
// e is exact, q0 + e/b is the exact quotient, and the quotient of two such short operands is either
// representable or at least 2^-13 ulp away from a rounding boundary, far more than the error of e*r.
// For fp32 operands, and for scales outside [2^-100, 2^100], the IEEE division is used directly.
struct BlockQ {
    float scale;
    float rcp;
    bool fast;
    __device__ __forceinline__ void set(float amax, bool short_mantissa) {
        scale = amax;
        fast = short_mantissa && amax > 7.8886090522101181e-31f && amax < 1.2676506002282294e30f;
        rcp = fast ? __frcp_rn(amax) : 0.0f;
    }
    // returns fl32(127 * fl32(x / scale)) + magic, whose low byte is the int8 result
    __device__ __forceinline__ uint32_t q(float x) const {
        if (fast) {
            float q0 = __fmul_rn(x, rcp);
            float e = __fmaf_rn(-scale, q0, x);
            float y = __fmaf_rn(e, rcp, q0);
            return __float_as_uint(__fadd_rn(__fmul_rn(127.0f, y), kMagic));
        }
        if (scale == 0.0f) return 0u;                 // 0/0: the reference stores 0
        float z = __fmul_rn(127.0f, __fdiv_rn(x, scale));
        if (!(z == z)) return 0u;                     // NaN converts to 0 in the int8 store
        return __float_as_uint(__fadd_rn(z, kMagic));
    }
};

__device__ __forceinline__ uint32_t pack4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    // low bytes of a,b,c,d -> one word (a in byte 0)
    uint32_t ab = __byte_perm(a, b, 0x0040);
    uint32_t cd = __byte_perm(c, d, 0x0040);
    return __byte_perm(ab, cd, 0x5410);
}

// packed pairs of fp32 values (one 64-bit register), every operation rounded on its own
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void f2_bits(uint64_t v, uint32_t& lo, uint32_t& hi) { asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

}  // namespace bi8
