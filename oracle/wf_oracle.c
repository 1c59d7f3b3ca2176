/*
 * CPU oracle for the ternary BitLinear hot path, plain C.
 *
 * TEST INFRASTRUCTURE ONLY: linked by the tests, the smoke check and the
 * CPU-baseline leg of the benchmark; never by the shipped library.
 * Parity status: pinned (the golden-vector tests compare these functions with
 * outputs of the reference's own code on seeded inputs).
 *
 * Each function cites the reference file it restates (paths inside the
 * reference project).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* round an fp32 value to the nearest bfloat16, ties to even; result as fp32 */
static inline float bf16_rn(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u = (u + 0x7fffu + lsb) & 0xffff0000u;
    float r;
    memcpy(&r, &u, 4);
    return r;
}

int wfo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* packages/training/src/wrinklefree/quantization/weight_quant.py:52 and :59-70
 * absmean with an fp64 sum, rounded once to fp32, clamped below by eps. */
float wfo_absmean(const float* w, int64_t n, float eps) {
    double s = 0.0;
#pragma omp parallel for reduction(+ : s) schedule(static)
    for (int64_t i = 0; i < n; ++i) s += fabs((double)w[i]);
    float m = n ? (float)(s / (double)n) : 0.0f;
    return m < eps ? eps : m;
}

/* weight_quant.py:53-54: codes = clamp(rint(w / scale), -1, 1), fp32 division,
 * round-half-even (the default FP environment). */
void wfo_ternarize(const float* w, int64_t n, float scale, int8_t* codes) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float q = nearbyintf(w[i] / scale);
        q = q < -1.f ? -1.f : (q > 1.f ? 1.f : q);
        codes[i] = (int8_t)q;
    }
}

/* The GPU layout of the library: row-major [N, K/4] bytes; in every 32-bit
 * little-endian word byte b, bit pair j holds weight k0 + 4*j + b, stored as
 * code = w + 1. */
void wfo_pack_wf16(const int8_t* codes, int64_t N, int64_t K, uint8_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const int8_t* c = codes + n * K;
        uint8_t* o = out + n * (K / 4);
        for (int64_t wd = 0; wd < K / 16; ++wd)
            for (int b = 0; b < 4; ++b) {
                uint8_t v = 0;
                for (int j = 0; j < 4; ++j) v |= (uint8_t)((c[wd * 16 + 4 * j + b] + 1) << (2 * j));
                o[wd * 4 + b] = v;
            }
    }
}

/* I2_S block layout, packages/inference/scripts/convert_to_sglkernel.py:96-111 */
void wfo_pack_i2s(const int8_t* codes, int64_t N, int64_t K, uint8_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int64_t blk = 0; blk < K / 128; ++blk)
            for (int j = 0; j < 32; ++j) {
                const int8_t* c = codes + n * K + blk * 128;
                out[n * (K / 4) + blk * 32 + j] = (uint8_t)(((c[j] + 1) << 6) | ((c[j + 32] + 1) << 4) |
                                                            ((c[j + 64] + 1) << 2) | (c[j + 96] + 1));
            }
}

/* packages/training/src/wrinklefree/models/bitlinear.py:79-82, per token.
 * mode 0: fp32 arithmetic.  mode 1: every intermediate rounded to bfloat16 as
 * torch does for a bf16 input.  x holds M*K fp32 values (already representable
 * in the mode's type).  scale[m] receives the rounded multiplier 127/absmax. */
void wfo_act_quant(const float* x, int64_t M, int64_t K, int mode, float eps, int8_t* q, float* scale) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        const float* r = x + m * K;
        float mx = 0.f;
        for (int64_t k = 0; k < K; ++k) {
            float a = fabsf(r[k]);
            if (a > mx) mx = a;
        }
        if (mx < eps) mx = eps;
        if (mode == 1) mx = bf16_rn(mx);
        /* torch evaluates `127.0 / t` as t.reciprocal() * 127.0: two roundings */
        float s = 1.0f / mx;
        if (mode == 1) s = bf16_rn(s);
        s = s * 127.0f;
        if (mode == 1) s = bf16_rn(s);
        scale[m] = s;
        for (int64_t k = 0; k < K; ++k) {
            float v = r[k] * s;
            if (mode == 1) v = bf16_rn(v);
            v = nearbyintf(v);
            v = v < -128.f ? -128.f : (v > 127.f ? 127.f : v);
            q[m * K + k] = (int8_t)v;
        }
    }
}

/* exact integer contraction acc[m,n] = sum_k q[m,k] * codes[n,k] */
void wfo_int_gemm(const int8_t* q, const int8_t* codes, int64_t M, int64_t N, int64_t K, int32_t* acc) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const int8_t* c = codes + n * K;
        for (int64_t m = 0; m < M; ++m) {
            const int8_t* a = q + m * K;
            int32_t s = 0;
            for (int64_t k = 0; k < K; ++k) s += (int32_t)a[k] * (int32_t)c[k];
            acc[m * N + n] = s;
        }
    }
}

/* y = (float(acc) * (1/scale[m])) * w_scale + bias[n]; the order is part of
 * the contract. */
void wfo_rescale(const int32_t* acc, const float* act_scale, float w_scale, const float* bias, int64_t M,
                 int64_t N, float* y) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        float inv = 1.0f / act_scale[m];
        for (int64_t n = 0; n < N; ++n) {
            float v = ((float)acc[m * N + n] * inv) * w_scale;
            if (bias) v += bias[n];
            y[m * N + n] = v;
        }
    }
}

/* The contraction on WF16-packed weights, used as the timed scalar port:
 * acc[m,n] = sum_k q[m,k] * (code[n,k] - 1). */
void wfo_gemm_wf16(const int8_t* q, const uint8_t* packed, int64_t M, int64_t N, int64_t K, int32_t* acc) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint32_t* wr = (const uint32_t*)(packed + n * (K / 4));
        for (int64_t m = 0; m < M; ++m) {
            const int8_t* a = q + m * K;
            int32_t s = 0;
            for (int64_t wd = 0; wd < K / 16; ++wd) {
                uint32_t w = wr[wd];
                for (int j = 0; j < 4; ++j)
                    for (int b = 0; b < 4; ++b) {
                        int c = (int)((w >> (8 * b + 2 * j)) & 3u) - 1;
                        s += c * (int32_t)a[wd * 16 + 4 * j + b];
                    }
            }
            acc[m * N + n] = s;
        }
    }
}
