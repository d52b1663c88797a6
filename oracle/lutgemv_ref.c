/*
 * CPU restatement of the reference's five LUT-GEMV kernels.  TEST INFRASTRUCTURE
 * ONLY: it is the checker for the CUDA library and is never linked into it.
 *
 * Each function follows the arithmetic of one kernel of the reference's
 * lut_gemm/mv_fp16_bias.hpp, with two deliberate differences: sums are carried
 * in double instead of fp16, and the K/32-way atomic split-K becomes a plain
 * loop.  What is kept exactly is the data layout and the index conventions:
 *   - packed planes  uint32 W[K/32][q][N]          (hpp:52, 86-90)
 *   - table index bit i set  => +x[8c+i], clear => -x[8c+i]   (hpp:19-45)
 *   - byte j of word kk indexes the table of chunk 4*kk+j     (hpp:86-90)
 *   - results are ADDED to what `out` already holds            (hpp:101)
 * fp16 operands are passed as IEEE binary16 bit patterns (uint16_t).
 *
 * Parity status: pinned indirectly — the test-suite checks these functions
 * against the numpy dequantise oracle, which is itself checked against outputs
 * of the reference's Python stored under tests/golden.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* 256-entry table of one chunk: hpp:19-45. */
static void build_table(const uint16_t *x8, double *lut) {
    float v[8];
    for (int i = 0; i < 8; i++) v[i] = half_to_float(x8[i]);
    for (int e = 0; e < 256; e++) {
        double s = 0.0;
        for (int i = 0; i < 8; i++) s += ((e >> i) & 1) ? v[i] : -v[i];
        lut[e] = s;
    }
}

static double *all_tables(const uint16_t *x, int K) {
    double *luts = (double *)malloc((size_t)(K / 8) * 256 * sizeof(double));
    if (!luts) return NULL;
    for (int c = 0; c < K / 8; c++) build_table(x + 8 * c, luts + (size_t)c * 256);
    return luts;
}

/* hpp:498-579  _nqmv_bias_shift_mulq : alpha fp16 [K/g][q][N]. */
int ref_shift_scale(float *out, const uint32_t *W, const uint16_t *alpha, const uint16_t *x,
                    int N, int K, int q, int num_groups) {
    if (K % 32 || num_groups <= 0 || K % num_groups) return -1;
    int g = K / num_groups;
    double *luts = all_tables(x, K);
    if (!luts) return -2;
    for (int n = 0; n < N; n++) {
        double acc = 0.0;
        for (int kk = 0; kk < K / 32; kk++) {
            int grp = (kk * 32) / g;
            for (int b = 0; b < q; b++) {
                uint32_t w = W[((size_t)kk * q + b) * N + n];
                double part = 0.0;
                for (int j = 0; j < 4; j++) part += luts[(size_t)(4 * kk + j) * 256 + ((w >> (8 * j)) & 255u)];
                acc += (double)half_to_float(alpha[((size_t)grp * q + b) * N + n]) * part;
            }
        }
        out[n] += (float)acc;
    }
    free(luts);
    return 0;
}

/* hpp:8-103  _nqmv_bias : alpha, q_bias fp16 [K/g][N]; plane b scaled by alpha / 2^(b+1);
 * q_bias multiplies the plain sum of the tile's activations (table entry 255). */
int ref_compute(float *out, const uint32_t *W, const uint16_t *alpha, const uint16_t *q_bias,
                const uint16_t *x, int N, int K, int q, int num_groups) {
    if (K % 32 || num_groups <= 0 || K % num_groups) return -1;
    int g = K / num_groups;
    double *luts = all_tables(x, K);
    if (!luts) return -2;
    for (int n = 0; n < N; n++) {
        double acc = 0.0;
        for (int kk = 0; kk < K / 32; kk++) {
            int grp = (kk * 32) / g;
            double xsum = 0.0;
            for (int j = 0; j < 4; j++) xsum += luts[(size_t)(4 * kk + j) * 256 + 255];
            acc += (double)half_to_float(q_bias[(size_t)grp * N + n]) * xsum;
            double a = half_to_float(alpha[(size_t)grp * N + n]);
            for (int b = 0; b < q; b++) {
                a *= 0.5;
                uint32_t w = W[((size_t)kk * q + b) * N + n];
                double part = 0.0;
                for (int j = 0; j < 4; j++) part += luts[(size_t)(4 * kk + j) * 256 + ((w >> (8 * j)) & 255u)];
                acc += a * part;
            }
        }
        out[n] += (float)acc;
    }
    free(luts);
    return 0;
}

/* Multiplier decoders for the three block kernels. */
static double mult_f16(const void *alpha, size_t idx) { return half_to_float(((const uint16_t *)alpha)[idx]); }
static double mult_u16(const void *alpha, size_t idx) { /* hpp:294-297 */
    unsigned a = ((const uint16_t *)alpha)[idx];
    return (double)(1u << (a & 7u)) + (double)(1u << ((a >> 3) & 7u)) + (double)(1u << ((a >> 6) & 7u));
}
static double mult_i8x3(const void *alpha, size_t idx) { /* hpp:335-340, 473-482; -128 = no term */
    const int8_t *a = (const int8_t *)alpha + idx * 3;
    double m = 0.0;
    for (int t = 0; t < 3; t++) if (a[t] != -128) m += ldexp(1.0, a[t]);
    return m;
}

/* hpp:105-220 / 223-328 / 342-495 : alpha [K/8][q][N/gs]; x [M][K]; out [M][N]. */
static int ref_block_generic(float *out, const uint32_t *W, const void *alpha, const uint16_t *x,
                             int M, int N, int K, int q, int num_groups,
                             double (*mult)(const void *, size_t)) {
    if (K % 32 || num_groups <= 0 || N % num_groups) return -1;
    int gs = N / num_groups;
    for (int m = 0; m < M; m++) {
        double *luts = all_tables(x + (size_t)m * K, K);
        if (!luts) return -2;
        for (int n = 0; n < N; n++) {
            int ng = n / gs;
            double acc = 0.0;
            for (int kk = 0; kk < K / 32; kk++) {
                for (int b = 0; b < q; b++) {
                    uint32_t w = W[((size_t)kk * q + b) * N + n];
                    for (int j = 0; j < 4; j++) {
                        size_t aidx = ((size_t)(4 * kk + j) * q + b) * num_groups + ng;
                        acc += mult(alpha, aidx) * luts[(size_t)(4 * kk + j) * 256 + ((w >> (8 * j)) & 255u)];
                    }
                }
            }
            out[(size_t)m * N + n] += (float)acc;
        }
        free(luts);
    }
    return 0;
}

int ref_block(float *out, const uint32_t *W, const uint16_t *alpha, const uint16_t *x,
              int M, int N, int K, int q, int num_groups) {
    return ref_block_generic(out, W, alpha, x, M, N, K, q, num_groups, mult_f16);
}
int ref_block_shift(float *out, const uint32_t *W, const uint16_t *alpha, const uint16_t *x,
                    int M, int N, int K, int q, int num_groups) {
    return ref_block_generic(out, W, alpha, x, M, N, K, q, num_groups, mult_u16);
}
int ref_block_shift_int8(float *out, const uint32_t *W, const int8_t *alpha, const uint16_t *x,
                         int M, int N, int K, int q, int num_groups) {
    return ref_block_generic(out, W, alpha, x, M, N, K, q, num_groups, mult_i8x3);
}
