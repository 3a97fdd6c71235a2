/* Plain-C restatement of the reference's blockwise-int8 path.  TEST INFRASTRUCTURE ONLY:
 * it is a second, independent checker next to blockwise_int8_oracle.py and the timed
 * multi-threaded CPU baseline; the shipped library never links or calls it.
 *
 * Each function cites the reference lines it follows (paths inside the reference project).
 * Compile with IEEE semantics only: no -ffast-math, and -ffp-contract=off so that the
 * separate fp32 multiply/divide/add steps of the reference are not fused.
 *
 *   gcc -O2 -fopenmp -ffp-contract=off -fPIC -shared -o libbi8_oracle.so bi8_oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even fp32 -> bf16 (NaN kept quiet) */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float load_elem(const void* x, int dtype, size_t i) {
    /* dtype: 0 = bf16 (as uint16), 1 = fp32 */
    return dtype == 0 ? bf16_to_f32(((const uint16_t*)x)[i]) : ((const float*)x)[i];
}

/* quantize_block_rowwise: triton_functions.py:382-406 (kernel), 411-423 (wrapper).
 * x [M,K] row-major, q [M,K] int8, s [ceil(K/B), M] fp32 (transposed). */
void bi8o_quantize_rowwise(const void* x, int dtype, int8_t* q, float* s, long M, long K, long B) {
    long nb = (K + B - 1) / B;
#pragma omp parallel for schedule(static)
    for (long m = 0; m < M; ++m) {
        for (long j = 0; j < nb; ++j) {
            long lo = j * B, hi = lo + B < K ? lo + B : K;
            float mx = 0.0f;                                   /* tail counts as zeros: 398-401 */
            for (long k = lo; k < hi; ++k) {
                float a = fabsf(load_elem(x, dtype, (size_t)m * K + k));
                if (a > mx) mx = a;
            }
            s[(size_t)j * M + m] = mx;                         /* line 404, stride M */
            for (long k = lo; k < hi; ++k) {
                float v = load_elem(x, dtype, (size_t)m * K + k);
                volatile float y = v / mx;                     /* fp32 divide, line 402 */
                volatile float z = 127.0f * y;                 /* separate fp32 multiply */
                float r = nearbyintf(z);                       /* llrint: round half to even */
                q[(size_t)m * K + k] = (r != r) ? 0 : (int8_t)(long)r;   /* NaN (0/0) stores 0 */
            }
        }
    }
}

/* dequantize_block_rowwise: triton_functions.py:467-490, line 487: max_val * x * inv_127.
 * out_dtype: 0 = bf16, 1 = fp32. */
void bi8o_dequantize_rowwise(const int8_t* q, const float* s, void* out, int out_dtype,
                             long M, long K, long B) {
    const float inv127 = (float)(1.0 / 127);
#pragma omp parallel for schedule(static)
    for (long m = 0; m < M; ++m) {
        for (long k = 0; k < K; ++k) {
            volatile float t = s[(size_t)(k / B) * M + m] * (float)q[(size_t)m * K + k];
            float v = t * inv127;
            if (out_dtype == 0) ((uint16_t*)out)[(size_t)m * K + k] = f32_to_bf16(v);
            else ((float*)out)[(size_t)m * K + k] = v;
        }
    }
}

/* int8_matmul_block64_rowwise_dequantize: triton_functions.py:69-139, accumulation line 120.
 * a [M,K] int8 row-major; bt [N,K] int8 row-major (the reference's b is bt transposed);
 * sx [nb,M], sw [nb,N]; acc_out [M,N] fp32 (the accumulator before the output cast). */
void bi8o_gemm_acc(const int8_t* a, const int8_t* bt, const float* sx, const float* sw,
                   float* acc_out, long M, long N, long K, long B) {
    long nb = (K + B - 1) / B;
    const float divf = (float)(1.0 / (127.0 * 127.0));
#pragma omp parallel for schedule(static) collapse(2)
    for (long m = 0; m < M; ++m) {
        for (long n = 0; n < N; ++n) {
            float acc = 0.0f;
            for (long j = 0; j < nb; ++j) {
                long lo = j * B, hi = lo + B < K ? lo + B : K;
                int32_t p = 0;
                for (long k = lo; k < hi; ++k)
                    p += (int32_t)a[(size_t)m * K + k] * (int32_t)bt[(size_t)n * K + k];
                volatile float t0 = (float)p * divf;
                volatile float t1 = sx[(size_t)j * M + m] * t0;
                volatile float t2 = sw[(size_t)j * N + n] * t1;
                acc = acc + t2;
            }
            acc_out[(size_t)m * N + n] = acc;
        }
    }
}

/* exact int32 block partial sums, out [nb, M, N] (triton_functions.py:115) */
void bi8o_gemm_partials(const int8_t* a, const int8_t* bt, int32_t* out,
                        long M, long N, long K, long B) {
    long nb = (K + B - 1) / B;
#pragma omp parallel for schedule(static) collapse(2)
    for (long j = 0; j < nb; ++j) {
        for (long m = 0; m < M; ++m) {
            long lo = j * B, hi = lo + B < K ? lo + B : K;
            for (long n = 0; n < N; ++n) {
                int32_t p = 0;
                for (long k = lo; k < hi; ++k)
                    p += (int32_t)a[(size_t)m * K + k] * (int32_t)bt[(size_t)n * K + k];
                out[((size_t)j * M + m) * N + n] = p;
            }
        }
    }
}
