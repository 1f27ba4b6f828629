/* CPU oracle for the fp16-in / fp32-accumulate GEMM and the attention forward.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against (tests, the smoke check and the benchmark's CPU-baseline
 * leg).  Nothing in the product library links, loads or calls it.
 *
 * Every function restates, in plain C, the arithmetic of the reference
 * (akeley98/spork); the citation beside each function names the reference
 * file and lines it follows.
 *
 * Pinning status:
 *   - GEMM: pinned on a GPU box by running the reference's own oracle kernel
 *     (gemm/gemm_baseline.cu, compiled unmodified into oracle/_ref) on the
 *     same fp16-representable inputs: results must agree bit for bit, since
 *     both accumulate in fp32 with k ascending and every fp16*fp16 product is
 *     exact in fp32.  Known-answer cases (identity x tiled_numbers) pin it on
 *     the CPU as well.
 *   - Attention: pinned against vectors generated here by executing the
 *     reference's simple_attn (torch_attn.py:11-16) on torch CPU; the vectors
 *     and their generator live in tests/golden/.
 *   - Fixture generators (pcg3d, test-data codes): the reference's generator is a
 *     device function inside gemm/gemm_test.cu, which cannot be compiled here
 *     (it includes generated headers); parity of the hash itself is pinned by
 *     the published test vectors of the PCG3D hash construction only through
 *     self-consistency between this file and the CUDA generator.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* fp16 <-> fp32, round-to-nearest-even, bit exact with __float2half_rn.      */

static inline float half_bits_to_float(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            /* subnormal: normalise */
            int shift = 0;
            while ((man & 0x400u) == 0) {
                man <<= 1;
                ++shift;
            }
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline uint16_t float_to_half_bits(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u : 0u));
    }
    if (x >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (x < 0x33000001u) { /* <= 2^-25 rounds to zero (ties-to-even at exactly 2^-25) */
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(x >> 23) - 127;
    uint32_t man = (x & 0x7FFFFFu) | 0x800000u;
    uint32_t shift;
    int32_t hexp;
    if (exp < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - exp));
        hexp = 0;
    } else {
        shift = 13;
        hexp = exp + 15;
    }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) {
        ++q;
    }
    uint32_t out;
    if (hexp == 0) {
        out = q; /* may carry into exponent 1: still the right encoding */
    } else {
        out = ((uint32_t)hexp << 10) + (q - 0x400u); /* carry bumps exponent */
    }
    return (uint16_t)(sign | out);
}

ORACLE_API float spork_oracle_half_to_float(uint16_t h) { return half_bits_to_float(h); }
ORACLE_API uint16_t spork_oracle_float_to_half(float f) { return float_to_half_bits(f); }

/* bfloat16 <-> fp32 (round to nearest even), the element type of the reference's attention interface. */
static inline float bf16_bits_to_float(uint16_t h)
{
    const uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline uint16_t float_to_bf16_bits(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) {
        return (uint16_t)((x >> 16) | 0x40u); /* quiet NaN */
    }
    x += 0x7FFFu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}

ORACLE_API float spork_oracle_bf16_to_float(uint16_t h) { return bf16_bits_to_float(h); }
ORACLE_API uint16_t spork_oracle_float_to_bf16(float f) { return float_to_bf16_bits(f); }

/* ------------------------------------------------------------------------- */
/* Position hash.  Follows gemm/gemm_test.cu:34-53 (the PCG3D hash of         */
/* Jarzynski & Olano, folded to 64 bits the way the reference folds it).      */

ORACLE_API uint64_t spork_oracle_pcg3d(uint32_t x, uint32_t y, uint32_t z)
{
    x = x * 1664525u + 1013904223u;
    y = y * 1664525u + 1013904223u;
    z = z * 1664525u + 1013904223u;
    x += y * z;
    y += z * x;
    z += x * y;
    x ^= x >> 16;
    y ^= y >> 16;
    z ^= z >> 16;
    x += y * z;
    y += z * x;
    z += x * y;
    return (uint64_t)x ^ ((uint64_t)y << 12) ^ ((uint64_t)z << 24);
}

/* Test-data codes.  0..2 are the reference's (gemm/gemm_test.h:6-11); 3 and 4
 * are the seeded distributions the headline configurations use. */
enum {
    SPORK_DATA_RANDOM = 0,
    SPORK_DATA_IDENTITY = 1,
    SPORK_DATA_TILED_NUMBERS = 2,
    SPORK_DATA_UNIFORM_PM1 = 3,
    SPORK_DATA_NORMAL = 4,
    SPORK_DATA_NORMAL_BM = 5,
};

/* One fixture element at logical coordinate (x, y).
 * Codes 0..2 follow gemm/gemm_test.cu:66-91 with T = fp16: integer values are
 * rounded to fp16 once; the sparse random value u^4 is formed in fp32 and then
 * rounded once.  Code 3: u = (hash & 0xFFFFFF) * 2^-23 - 1, exact in fp32.
 * Code 4: Irwin-Hall sum of twelve 24-bit hashed uniforms minus 6 (mean 0,
 * variance 1, integer arithmetic so that CPU and GPU agree bit for bit). */
static inline uint16_t fixture_value(uint32_t x, uint32_t y, int code, uint32_t seed)
{
    switch (code) {
    case SPORK_DATA_IDENTITY:
        return x == y ? 0x3C00u : 0u;
    case SPORK_DATA_TILED_NUMBERS:
        return float_to_half_bits((float)((x % 64u) + 100u * (y % 64u)));
    case SPORK_DATA_UNIFORM_PM1: {
        const uint32_t bits = (uint32_t)(spork_oracle_pcg3d(x, y, seed) & 0xFFFFFFu);
        return float_to_half_bits((float)bits * (1.0f / 8388608.0f) - 1.0f);
    }
    case SPORK_DATA_NORMAL: {
        uint32_t sum = 0;
        for (uint32_t i = 0; i < 12u; ++i) {
            sum += (uint32_t)(spork_oracle_pcg3d(x, y, seed + 0x9E3779B9u * i) & 0xFFFFFFu);
        }
        /* sum < 12 * 2^24; (sum - 6 * 2^24) * 2^-24 is exact in fp32 only up to
         * 24 significant bits, so round once through double. */
        const double v = ((double)sum - 6.0 * 16777216.0) * (1.0 / 16777216.0);
        return float_to_half_bits((float)v);
    }
    case SPORK_DATA_NORMAL_BM: {
        /* Box-Muller on two hashed 24-bit uniforms, as the device generator does; the C library's logf /
         * cosf may differ from the device's in the last bit, so this code is statistically, not bitwise,
         * the same fixture (parity tests read the device's bits back instead). */
        const uint64_t h = spork_oracle_pcg3d(x, y, seed);
        const float u1 = ((float)(uint32_t)(h & 0xFFFFFFu) + 1.0f) * (1.0f / 16777216.0f);
        const float u2 = (float)(uint32_t)((h >> 24) & 0xFFFFFFu) * (1.0f / 16777216.0f);
        return float_to_half_bits(sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2));
    }
    case SPORK_DATA_RANDOM:
    default: {
        const uint64_t randbits = spork_oracle_pcg3d(x, y, 20010106u);
        if (randbits % 100000u == 0) {
            return float_to_half_bits(1000.0f);
        }
        if (randbits % 4u != 0u) {
            return 0u;
        }
        float v = (float)(spork_oracle_pcg3d(x, y, 19980724u) % 1000000u) * 1e-6f;
        v = (v * v) * (v * v);
        return float_to_half_bits(v);
    }
    }
}

/* Fill a rows x cols row-major fp16 matrix.  transpose_rule swaps the logical
 * coordinate fed to the hash, exactly as gemm/gemm_test.cu:55-65 does, so a
 * matrix and its stored transpose hold the same logical values. */
ORACLE_API void spork_oracle_fill_f16(uint16_t* out, uint32_t rows, uint32_t cols, int code, uint32_t seed,
                                      int transpose_rule)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        for (uint32_t c = 0; c < cols; ++c) {
            const uint32_t x = transpose_rule ? (uint32_t)r : c;
            const uint32_t y = transpose_rule ? c : (uint32_t)r;
            out[(size_t)r * cols + c] = fixture_value(x, y, code, seed);
        }
    }
}

/* ------------------------------------------------------------------------- */
/* GEMM.  C[m,n] = sum_k A[m,k] * B[n,k]; A is M x K row-major, B is stored    */
/* N x K row-major (the harness's "b_col_major = 1" operand,                   */
/* gemm/gemm_test.cu:305), C is M x N row-major fp32.                          */
/*                                                                             */
/* Loop structure of docs/nyc25.py:34-55 (accum = 0; for k: accum += a*b;      */
/* C[m,n] = accum) with fp32 accumulation in ascending k as in                 */
/* gemm/gemm_baseline.cu:74-83.  B is first widened into a K x N fp32 panel    */
/* (the layout nyc25_gemm_cpu takes), cut into column panels, so that a small  */
/* block of outputs shares one pass over k; each output element still sees     */
/* exactly the scalar recurrence above.                                        */

#define NB 16 /* output columns per panel */
#define MB 4  /* output rows sharing one pass over a panel */

ORACLE_API int spork_oracle_gemm_f16f32(uint32_t M, uint32_t N, uint32_t K, const uint16_t* A, const uint16_t* B,
                                        float* C)
{
    if (M == 0 || N == 0) {
        return 0;
    }
    const size_t panels = ((size_t)N + NB - 1) / NB;
    const size_t Kp = K ? K : 1;
    /* Bt[panel][k][NB]: the K x N operand cut into NB-wide column panels. */
    float* Bt = (float*)calloc(panels * Kp * NB, sizeof(float));
    if (!Bt) {
        return 1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)N; ++n) {
        float* dst = Bt + ((size_t)n / NB) * Kp * NB + (size_t)n % NB;
        for (uint32_t k = 0; k < K; ++k) {
            dst[(size_t)k * NB] = half_bits_to_float(B[(size_t)n * K + k]);
        }
    }
    int failed = 0;
    const int64_t row_blocks = ((int64_t)M + MB - 1) / MB;
#pragma omp parallel
    {
        float* arows = (float*)calloc(Kp * MB, sizeof(float)); /* arows[k][MB] */
        if (!arows) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 2)
        for (int64_t mb = 0; mb < row_blocks; ++mb) {
            if (!arows) {
                continue;
            }
            const uint32_t m0 = (uint32_t)(mb * MB);
            const uint32_t mrows = M - m0 < MB ? M - m0 : MB;
            for (uint32_t i = 0; i < MB; ++i) {
                for (uint32_t k = 0; k < K; ++k) {
                    arows[(size_t)k * MB + i] = i < mrows ? half_bits_to_float(A[(size_t)(m0 + i) * K + k]) : 0.0f;
                }
            }
            for (size_t pn = 0; pn < panels; ++pn) {
                float acc[MB][NB];
                for (int i = 0; i < MB; ++i) {
                    for (int j = 0; j < NB; ++j) {
                        acc[i][j] = 0.0f;
                    }
                }
                const float* bp = Bt + pn * Kp * NB;
                for (uint32_t k = 0; k < K; ++k) {
                    const float* b = bp + (size_t)k * NB;
                    const float* a = arows + (size_t)k * MB;
                    for (int i = 0; i < MB; ++i) {
                        for (int j = 0; j < NB; ++j) {
                            acc[i][j] += a[i] * b[j];
                        }
                    }
                }
                for (uint32_t i = 0; i < mrows; ++i) {
                    for (int j = 0; j < NB && pn * NB + j < N; ++j) {
                        C[(size_t)(m0 + i) * N + pn * NB + j] = acc[i][j];
                    }
                }
            }
        }
        free(arows);
    }
    free(Bt);
    return failed;
}

/* The reference's own operand type: fp32 A (M x K) and B (stored N x K), fp32 accumulation, k ascending -
 * nyc25_gemm_cpu (docs/nyc25.py:13-56) on the harness layout.  tf32_mode says what happens to the operands
 * before the multiply: 0 = nothing (plain fp32, what gemm/gemm_baseline.cu computes), 1 = the low 13
 * mantissa bits are dropped (truncation to tf32), 2 = rounded to tf32, nearest with ties away from zero
 * (cvt.rna.tf32.f32).  tf32 x tf32 products are exact in fp32. */
static inline float to_tf32(float x, int mode)
{
    uint32_t u;
    memcpy(&u, &x, 4);
    if (mode == 2 && (u & 0x7F800000u) != 0x7F800000u) {
        u += 0x1000u;
    }
    if (mode != 0) {
        u &= 0xFFFFE000u;
    }
    memcpy(&x, &u, 4);
    return x;
}

ORACLE_API int spork_oracle_gemm_f32(uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B, float* C,
                                     int tf32_mode)
{
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t m = 0; m < (int64_t)M; ++m) {
        for (uint32_t n = 0; n < N; ++n) {
            float acc = 0.0f;
            for (uint32_t k = 0; k < K; ++k) {
                /* the product is formed exactly (double) and rounded once to fp32, as an FMA would not
                 * round it at all for tf32 operands and as fp32 multiply does for plain operands */
                const float a = to_tf32(A[(size_t)m * K + k], tf32_mode);
                const float b = to_tf32(B[(size_t)n * K + k], tf32_mode);
                acc = tf32_mode ? (float)((double)acc + (double)a * (double)b) : acc + a * b;
            }
            C[(size_t)m * N + n] = acc;
        }
    }
    return 0;
}

/* Same contraction with fp64 accumulation: bounds the oracle's own rounding. */
ORACLE_API int spork_oracle_gemm_f16f64(uint32_t M, uint32_t N, uint32_t K, const uint16_t* A, const uint16_t* B,
                                        double* C)
{
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t m = 0; m < (int64_t)M; ++m) {
        for (uint32_t n = 0; n < N; ++n) {
            double acc = 0.0;
            for (uint32_t k = 0; k < K; ++k) {
                acc += (double)half_bits_to_float(A[(size_t)m * K + k]) *
                       (double)half_bits_to_float(B[(size_t)n * K + k]);
            }
            C[(size_t)m * N + n] = acc;
        }
    }
    return 0;
}

/* Rows [m0, m0+rows) of the same product: used to check samples of a large C. */
ORACLE_API int spork_oracle_gemm_f16f32_rows(uint32_t M, uint32_t N, uint32_t K, const uint16_t* A,
                                             const uint16_t* B, uint32_t m0, uint32_t rows, float* C_rows)
{
    if (m0 > M || rows > M - m0) {
        return 2;
    }
    return spork_oracle_gemm_f16f32(rows, N, K, A + (size_t)m0 * K, B, C_rows);
}

/* ------------------------------------------------------------------------- */
/* Error metrics.                                                              */

/* max |c - ref| / (max|A| * max|B| * K * 2^-10): the acceptance metric of the
 * headline configurations (must be <= 1). */
ORACLE_API double spork_oracle_normalised_error(uint64_t count, const float* c, const float* ref, double max_abs_a,
                                                double max_abs_b, uint32_t K)
{
    double worst = 0.0;
    for (uint64_t i = 0; i < count; ++i) {
        double d = fabs((double)c[i] - (double)ref[i]);
        if (!(d == d)) {
            return INFINITY;
        }
        if (d > worst) {
            worst = d;
        }
    }
    const double denom = max_abs_a * max_abs_b * (double)(K ? K : 1) * (1.0 / 1024.0);
    return denom > 0 ? worst / denom : (worst > 0 ? INFINITY : 0.0);
}

/* The reference's comparator (gemm/gemm_test.cu:131-154): an element passes iff
 * the two values have the same sign (no NaN/inf) and max/min < 1 + 1/32, or
 * both are zero.  Returns the packed (row << 32 | col) of the first failure in
 * row-major order, or UINT64_MAX when everything passes. */
ORACLE_API uint64_t spork_oracle_ratio_compare(const float* a_mat, const float* b_mat, uint32_t rows, uint32_t cols)
{
    for (uint32_t y = 0; y < rows; ++y) {
        for (uint32_t x = 0; x < cols; ++x) {
            float a = a_mat[(size_t)y * cols + x];
            float b = b_mat[(size_t)y * cols + x];
            int correct = a * b >= 0.0f;
            if (correct) {
                a = fabsf(a);
                b = fabsf(b);
                const float lo = fminf(a, b);
                const float hi = fmaxf(a, b);
                correct = hi == 0 || hi / lo < (1.0f + 1 / 32.0f);
            }
            if (!correct) {
                return ((uint64_t)y << 32) | x;
            }
        }
    }
    return UINT64_MAX;
}

/* ------------------------------------------------------------------------- */
/* Attention forward, one head at a time.  Follows torch_attn.py:11-16:        */
/*   S = Q K^T * scale ; P = softmax(S, rows) ; O = P V, all in fp32;          */
/* inputs are fp16 bits, the fp32 result is rounded to fp16 once at the end    */
/* (o16) and also returned unrounded (o32, may be NULL).                        */
/* Layout: [BH][S][D] row-major for q, k, v, o - each head is the reference's  */
/* single (N, d) problem (matrix_util.hpp:40-45).                              */

static int attn_any(int BH, int S, int D, const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* o16,
                    float* o32, float scale, int bf16, int causal);

ORACLE_API int spork_oracle_attn_f16(int BH, int S, int D, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                     uint16_t* o16, float* o32, float scale)
{
    return attn_any(BH, S, D, q, k, v, o16, o32, scale, 0, 0);
}

/* Same with bfloat16 bit patterns in and out (the reference interface's element type). */
ORACLE_API int spork_oracle_attn_bf16(int BH, int S, int D, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                      uint16_t* o16, float* o32, float scale)
{
    return attn_any(BH, S, D, q, k, v, o16, o32, scale, 1, 0);
}

/* Causal variant (an addition: the reference's simple_attn has no mask): query i attends to keys j <= i only,
 * i.e. the softmax and the sum run over the first i + 1 keys. */
ORACLE_API int spork_oracle_attn_ex(int BH, int S, int D, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                    uint16_t* o16, float* o32, float scale, int bf16, int causal)
{
    return attn_any(BH, S, D, q, k, v, o16, o32, scale, bf16, causal);
}

static int attn_any(int BH, int S, int D, const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* o16,
                    float* o32, float scale, int bf16, int causal)
{
    if (BH < 0 || S <= 0 || D <= 0) {
        return 2;
    }
    int failed = 0;
    const int64_t total = (int64_t)BH * S;
#pragma omp parallel
    {
        float* kf = (float*)malloc(sizeof(float) * (size_t)S * D);
        float* vf = (float*)malloc(sizeof(float) * (size_t)S * D);
        float* qrow = (float*)malloc(sizeof(float) * (size_t)D);
        float* p = (float*)malloc(sizeof(float) * (size_t)S);
        float* orow = (float*)malloc(sizeof(float) * (size_t)D);
        const int ok = kf && vf && qrow && p && orow;
        if (!ok) {
#pragma omp atomic write
            failed = 1;
        }
        int cur_head = -1; /* head whose K and V this thread holds widened to fp32 */
#pragma omp for schedule(static)
        for (int64_t t = 0; t < total; ++t) {
            if (!ok) {
                continue;
            }
            const int h = (int)(t / S);
            const int i = (int)(t % S);
            const size_t base = (size_t)h * S * D;
            if (h != cur_head) {
                for (size_t e = 0; e < (size_t)S * D; ++e) {
                    kf[e] = bf16 ? bf16_bits_to_float(k[base + e]) : half_bits_to_float(k[base + e]);
                    vf[e] = bf16 ? bf16_bits_to_float(v[base + e]) : half_bits_to_float(v[base + e]);
                }
                cur_head = h;
            }
            for (int d = 0; d < D; ++d) {
                qrow[d] = bf16 ? bf16_bits_to_float(q[base + (size_t)i * D + d])
                               : half_bits_to_float(q[base + (size_t)i * D + d]);
            }
            const int keys = causal ? i + 1 : S; /* keys this query attends to */
            float row_max = -INFINITY;
            for (int j = 0; j < keys; ++j) {
                float acc = 0.0f;
                for (int d = 0; d < D; ++d) {
                    acc += qrow[d] * kf[(size_t)j * D + d];
                }
                acc *= scale;
                p[j] = acc;
                if (acc > row_max) {
                    row_max = acc;
                }
            }
            float denom = 0.0f;
            for (int j = 0; j < keys; ++j) {
                p[j] = expf(p[j] - row_max);
                denom += p[j];
            }
            for (int d = 0; d < D; ++d) {
                orow[d] = 0.0f;
            }
            for (int j = 0; j < keys; ++j) {
                const float pj = p[j] / denom;
                for (int d = 0; d < D; ++d) {
                    orow[d] += pj * vf[(size_t)j * D + d];
                }
            }
            for (int d = 0; d < D; ++d) {
                if (o32) {
                    o32[base + (size_t)i * D + d] = orow[d];
                }
                if (o16) {
                    o16[base + (size_t)i * D + d] = bf16 ? float_to_bf16_bits(orow[d]) : float_to_half_bits(orow[d]);
                }
            }
        }
        free(kf);
        free(vf);
        free(qrow);
        free(p);
        free(orow);
    }
    return failed;
}

/* Number of OpenMP threads later calls use (launchers often export OMP_NUM_THREADS=1). */
ORACLE_API void spork_oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n >= 1) {
        omp_set_num_threads(n);
    }
#else
    (void)n;
#endif
}

ORACLE_API int spork_oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
