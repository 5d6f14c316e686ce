/*
 * CPU oracle, plain C: NVFP4 block-scaled dual GEMM / grouped GEMM.
 *
 * TEST INFRASTRUCTURE ONLY -- never linked into the shipped library.  It is an
 * independent restatement (no torch, no BLAS) of the reference's fp32
 * dequantise-then-matmul check, reading the *permuted* scale-factor buffers a
 * kernel receives:
 *   e2m1 table / nibble order   group_gemm/group_gemm_cute5_v2.py:4436-4457
 *   e4m3fn scale bytes          dual_gemm/reference.py:146-147
 *   permuted SF index map       dual_gemm/reference.py:181-188
 *   fp32 dequant + contraction  group_gemm/group_gemm_cute5_v2.py:3827-3829
 *   silu(r1)*r2 -> fp16         dual_gemm/reference.py:76
 * Parity pins: see the header of nvfp4_oracle.py; the tests compare this file
 * against that module and against the golden vectors.
 *
 * Build: gcc -O3 -shared -fPIC (see oracle/Makefile); single-threaded unless built with -fopenmp.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

float oracle_e4m3_to_f32(uint8_t v) {
    int e = (v >> 3) & 0xF, m = v & 7;
    float s = (v & 0x80) ? -1.0f : 1.0f;
    if (e == 0xF && m == 7) return NAN;
    if (e == 0) return s * ldexpf((float)m / 8.0f, -6);
    return s * ldexpf(1.0f + (float)m / 8.0f, e - 7);
}

/* fp32 -> fp16 bits, round to nearest even, overflow to inf (IEEE, like
 * torch's .to(float16)). */
uint16_t oracle_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);            /* NaN */
    if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);           /* >= 65520 -> inf */
    if (absx < 0x33000001u) return (uint16_t)sign;                        /* < 2^-25 (or tie) -> 0 */
    int exp = (int)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t half;
    if (exp < -14) {                                                       /* subnormal */
        int shift = -14 - exp + 13;
        uint32_t q = man >> shift, rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (q & 1))) q++;
        half = q;
    } else {
        uint32_t q = man >> 13, rem = man & 0x1FFFu;
        half = ((uint32_t)(exp + 15) << 10) + (q & 0x3FFu);
        if (rem > 0x1000u || (rem == 0x1000u && (q & 1))) half++;
    }
    return (uint16_t)(sign | half);
}

static inline size_t sf_off(int i, int j, int rest_k) {
    return ((size_t)(i / 128) * rest_k + j / 4) * 512 + (size_t)(i % 32) * 16 + ((i % 128) / 32) * 4 + (j % 4);
}

/* rows x K fp32 = e2m1(packed) * e4m3(sf_perm), one batch. */
void oracle_dequant(const uint8_t* packed, const uint8_t* sf_perm, int rows, int k, float* out) {
    int rest_k = (k / 16 + 3) / 4;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < rows; ++i) {
        const uint8_t* p = packed + (size_t)i * (k / 2);
        float* o = out + (size_t)i * k;
        for (int j = 0; j < k / 16; ++j) {
            float s = oracle_e4m3_to_f32(sf_perm[sf_off(i, j, rest_k)]);
            for (int t = 0; t < 8; ++t) {
                uint8_t byte = p[j * 8 + t];
                o[j * 16 + 2 * t] = kE2M1[byte & 0xF] * s;
                o[j * 16 + 2 * t + 1] = kE2M1[byte >> 4] * s;
            }
        }
    }
}

static void gemm_nt(const float* a, const float* b, int m, int n, int k, float* c) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            const float *x = a + (size_t)i * k, *y = b + (size_t)j * k;
            float acc[8] = {0};
            for (int t = 0; t < k; t += 8)
                for (int u = 0; u < 8; ++u) acc[u] += x[t + u] * y[t + u];
            c[(size_t)i * n + j] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
        }
}

/* One batch of the dual GEMM; c is fp16 bits [m, n] with row pitch ldc.
 * Returns 0, or -1 on allocation failure. */
int oracle_dual_gemm(const uint8_t* a, const uint8_t* b1, const uint8_t* b2, const uint8_t* sfa_perm,
                     const uint8_t* sfb1_perm, const uint8_t* sfb2_perm, uint16_t* c, int m, int n, int k,
                     long ldc) {
    float* da = malloc((size_t)m * k * 4);
    float* db = malloc((size_t)n * k * 4);
    float* r1 = malloc((size_t)m * n * 4);
    float* r2 = malloc((size_t)m * n * 4);
    if (!da || !db || !r1 || !r2) { free(da); free(db); free(r1); free(r2); return -1; }
    oracle_dequant(a, sfa_perm, m, k, da);
    oracle_dequant(b1, sfb1_perm, n, k, db);
    gemm_nt(da, db, m, n, k, r1);
    oracle_dequant(b2, sfb2_perm, n, k, db);
    gemm_nt(da, db, m, n, k, r2);
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            float x = r1[(size_t)i * n + j], y = r2[(size_t)i * n + j];
            float silu = x / (1.0f + expf(-x));
            c[(size_t)i * ldc + j] = oracle_f32_to_f16(silu * y);
        }
    free(da); free(db); free(r1); free(r2);
    return 0;
}

/* One group of the grouped GEMM (no activation). */
int oracle_gemm(const uint8_t* a, const uint8_t* b, const uint8_t* sfa_perm, const uint8_t* sfb_perm,
                uint16_t* c, int m, int n, int k, long ldc) {
    if (m == 0 || n == 0) return 0;
    float* da = malloc((size_t)m * k * 4);
    float* db = malloc((size_t)n * k * 4);
    float* r = malloc((size_t)m * n * 4);
    if (!da || !db || !r) { free(da); free(db); free(r); return -1; }
    oracle_dequant(a, sfa_perm, m, k, da);
    oracle_dequant(b, sfb_perm, n, k, db);
    gemm_nt(da, db, m, n, k, r);
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) c[(size_t)i * ldc + j] = oracle_f32_to_f16(r[(size_t)i * n + j]);
    free(da); free(db); free(r);
    return 0;
}
