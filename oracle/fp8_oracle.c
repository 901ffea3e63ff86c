/*
 * CPU oracle for the FP8 GEMM path.  TEST INFRASTRUCTURE ONLY: this file is the
 * checker that the CUDA library is compared against.  Nothing in the product
 * path links, imports or executes it; only the test-suite, the smoke check and
 * the benchmark's CPU-baseline leg do.
 *
 * It restates, in plain C, the arithmetic of the reference project
 * (xuezy-mmi/Tensor-Core-FP8):
 *
 *   - the operator contract of gemm::GEMM / gemm::GEMM4
 *     (GEMM/include/gemm.cuh:12-55): C[m][n] = sum_k A[m][k] * B[n][k] with
 *     A row-major M x K bytes, B "column-major K x N" = stored [N][K] bytes,
 *     C row-major M x N FP32;
 *   - the reference's CPU verification loop (GEMM/gemm_main.cpp:45-52): float
 *     accumulation in ascending k, one product at a time;
 *   - the reference's input generator MakeDenseMatrix
 *     (GEMM/include/bm_test_utils.h:131-143): uniform(-1,1) floats from a
 *     default-seeded std::default_random_engine, converted by the FP8
 *     constructor (round-to-nearest-even, saturate-to-finite);
 *   - the FP8 formats themselves, which the reference takes from the CUDA
 *     toolkit header cuda_fp8.h (call sites bm_test_utils.h:139 and
 *     gemm_main.cpp:48); the toolkit is a third-party dependency that is not
 *     part of the reference tree (CUDA 12.4 named in GEMM/makefile:1).
 *
 * Parity pin: every function below is checked (tests/test_oracle_*.py) against
 * fixtures under tests/golden/ that were produced by running the reference's
 * own code in place (its MakeDenseMatrix and its verification loop) and the
 * toolkit's host conversions; see tests/golden/make_golden.py.
 *
 * Format codes: 0 = e4m3 (1-4-3, bias 7, max 448, no infinity, 0x7F/0xFF NaN),
 *               1 = e5m2 (1-5-2, bias 15, max 57344, IEEE-like inf/NaN).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_E4M3 0
#define ORACLE_E5M2 1

/* ---- decode ------------------------------------------------------------- */

/* Value of one FP8 byte as a double (exact: every FP8 value is a double). */
double oracle_fp8_decode(uint8_t byte, int fmt)
{
    const int mant_bits = (fmt == ORACLE_E4M3) ? 3 : 2;
    const int exp_bits = 7 - mant_bits;
    const int bias = (fmt == ORACLE_E4M3) ? 7 : 15;
    const int sign = byte >> 7;
    const int e = (byte >> mant_bits) & ((1 << exp_bits) - 1);
    const int m = byte & ((1 << mant_bits) - 1);
    double v;
    if (fmt == ORACLE_E4M3) {
        if (e == 15 && m == 7) return NAN;
    } else {
        if (e == 31) return m ? NAN : (sign ? -INFINITY : INFINITY);
    }
    if (e == 0)
        v = ldexp((double)m, 1 - bias - mant_bits);
    else
        v = ldexp((double)((1 << mant_bits) | m), e - bias - mant_bits);
    return sign ? -v : v;
}

void oracle_fp8_decode_table(int fmt, double *out256)
{
    for (int i = 0; i < 256; ++i) out256[i] = oracle_fp8_decode((uint8_t)i, fmt);
}

/* ---- encode: round-to-nearest-even, saturate-to-finite ------------------ */

/*
 * float -> FP8 byte with the semantics of the toolkit's
 * __nv_cvt_float_to_fp8(x, __NV_SATFINITE, fmt), which is what the FP8
 * constructors used by the reference (bm_test_utils.h:139) perform:
 * ties to even, overflow and +-inf clamp to +-max finite, NaN stays NaN,
 * magnitudes at or below half the smallest subnormal become (signed) zero.
 */
uint8_t oracle_fp8_encode(float x, int fmt)
{
    const int mant_bits = (fmt == ORACLE_E4M3) ? 3 : 2;
    const int bias = (fmt == ORACLE_E4M3) ? 7 : 15;
    const uint8_t max_code = (fmt == ORACLE_E4M3) ? 0x7E : 0x7B;
    const double max_val = (fmt == ORACLE_E4M3) ? 448.0 : 57344.0;
    const int emin = 1 - bias; /* exponent of the smallest normal */
    uint32_t bits;
    memcpy(&bits, &x, sizeof bits);
    const uint8_t sign = (uint8_t)((bits >> 31) << 7);

    if (isnan(x)) {
        /* the toolkit canonicalises every NaN to +NaN with all mantissa bits set */
        return 0x7F;
    }
    double a = fabs((double)x);
    if (a == 0.0) return sign;

    /* Quantum of the target grid at this magnitude. */
    int e;
    (void)frexp(a, &e); /* a = f * 2^e, f in [0.5,1)  => floor(log2 a) = e-1 */
    int ex = e - 1;
    if (ex < emin) ex = emin; /* subnormal range shares the smallest normal's grid */
    const double quantum = ldexp(1.0, ex - mant_bits);
    double q = a / quantum; /* exact: power-of-two scaling */
    double r = nearbyint(q); /* default rounding mode = ties to even */
    double v = r * quantum;
    if (v > max_val) return (uint8_t)(sign | max_code);
    if (v == 0.0) return sign;

    /* Re-derive exponent/mantissa of the rounded value. */
    (void)frexp(v, &e);
    ex = e - 1;
    uint8_t code;
    if (ex < emin) {
        code = (uint8_t)(v / ldexp(1.0, emin - mant_bits));
    } else {
        int m = (int)(v / ldexp(1.0, ex - mant_bits)) - (1 << mant_bits);
        code = (uint8_t)(((ex + bias) << mant_bits) | m);
    }
    return (uint8_t)(sign | code);
}

void oracle_fp8_encode_array(const float *x, int64_t n, int fmt, uint8_t *out)
{
    for (int64_t i = 0; i < n; ++i) out[i] = oracle_fp8_encode(x[i], fmt);
}

/* ---- the reference's input generator ------------------------------------ */

/*
 * MakeDenseMatrix (bm_test_utils.h:131-143) restated: the engine is
 * std::default_random_engine, which in libstdc++ is minstd_rand0
 * (x <- 16807 x mod 2^31-1, default seed 1), drawn through
 * std::uniform_real_distribution<float>(-1, 1), i.e. one engine draw per
 * sample mapped by generate_canonical<float,24>: (draw - 1) / 2147483646 in
 * float arithmetic, clamped below 1, then scaled to (-1, 1).
 * The engine is passed BY VALUE in the reference, so every matrix restarts
 * the same stream; `state` is the engine state to start from (1 = default).
 */
void oracle_make_dense_uniform(int64_t count, int fmt, uint32_t state, uint8_t *out)
{
    uint64_t x = state;
    for (int64_t i = 0; i < count; ++i) {
        x = (x * 16807ULL) % 2147483647ULL;
        float sum = (float)(x - 1ULL);
        float ret = sum / 2147483646.0f;
        if (ret >= 1.0f) ret = nextafterf(1.0f, 0.0f);
        float sample = ret * (1.0f - (-1.0f)) + (-1.0f);
        out[i] = oracle_fp8_encode(sample, fmt);
    }
}

/* ---- seeded normal inputs used by the benchmark configurations ----------- */

static inline uint64_t splitmix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111CBULL;
    return z ^ (z >> 31);
}

/*
 * Counter-based N(0, sigma^2) sample for linear element index `idx` of the
 * tensor with the given seed (Box-Muller on two 24-bit uniforms from one
 * splitmix64 hash).  The device-side generator of the library uses the same
 * recipe; transcendental functions differ in the last ulp between host and
 * device, so tests treat the BYTES read back from the device as ground truth
 * and use this function only for distribution checks.
 */
float oracle_normal_sample(uint64_t seed, uint64_t idx, float sigma)
{
    uint64_t h = splitmix64(seed ^ splitmix64(idx));
    uint32_t u1 = (uint32_t)(h >> 40);          /* 24 bits */
    uint32_t u2 = (uint32_t)((h >> 16) & 0xFFFFFF);
    float f1 = ((float)u1 + 1.0f) * (1.0f / 16777216.0f); /* (0,1] */
    float f2 = (float)u2 * (1.0f / 16777216.0f);          /* [0,1) */
    float r = sqrtf(-2.0f * logf(f1));
    return sigma * r * cosf(6.28318530717958647692f * f2);
}

void oracle_fill_normal_fp8(uint8_t *out, int64_t n, int fmt, float sigma,
                            uint64_t seed, uint64_t index_offset)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i)
        out[i] = oracle_fp8_encode(oracle_normal_sample(seed, index_offset + (uint64_t)i, sigma), fmt);
}

/* ---- the reference's CPU GEMM ------------------------------------------- */

static void float_table(int fmt, float *t)
{
    for (int i = 0; i < 256; ++i) t[i] = (float)oracle_fp8_decode((uint8_t)i, fmt);
}

/*
 * gemm_main.cpp:45-52 restated: for each (m, n), a float accumulator that
 * starts at 0 and adds (float)A[m][k] * (float)B[n][k] for k = 0..K-1 in
 * order.  `threads` <= 1 runs exactly as the reference does (one thread);
 * larger values split the m loop over OpenMP threads (each output element is
 * still accumulated by one thread in the same order, so results are
 * bit-identical).  Rows m0..m1-1 and columns n0..n1-1 only (a bounded sample
 * of a larger problem when timing); C is addressed with leading dimension ldc
 * relative to (m0, n0).
 */
void oracle_gemm_ref_float_block(int M, int K, int N, const uint8_t *A, int fmt_a,
                                 const uint8_t *B, int fmt_b, float *C, int64_t ldc,
                                 int m0, int m1, int n0, int n1, int threads)
{
    float ta[256], tb[256];
    float_table(fmt_a, ta);
    float_table(fmt_b, tb);
    (void)M;
    (void)N;
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
#endif
    for (int m = m0; m < m1; ++m) {
        const uint8_t *a = A + (int64_t)m * K;
        for (int n = n0; n < n1; ++n) {
            const uint8_t *b = B + (int64_t)n * K;
            /* volatile-free but strictly sequential: no reassociation without -ffast-math */
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += ta[a[k]] * tb[b[k]];
            C[(int64_t)(m - m0) * ldc + (n - n0)] = acc;
        }
    }
}

void oracle_gemm_ref_float(int M, int K, int N, const uint8_t *A, int fmt_a,
                           const uint8_t *B, int fmt_b, float *C, int threads)
{
    oracle_gemm_ref_float_block(M, K, N, A, fmt_a, B, fmt_b, C, N, 0, M, 0, N, threads);
}

/* ---- FP64 oracle with the per-element tolerance denominator -------------- */

/*
 * C64[m][n] = sum_k a*b and S[m][n] = sum_k |a*b| in double over the block
 * rows m0..m1-1 x columns n0..n1-1 (outputs are (m1-m0) x (n1-n0), row-major).
 * Products of two FP8 values are exact in double and the sums of up to 2^31
 * such products carry a relative error below 2^-21 of S, far inside the 1e-3*S
 * tolerance they are used for.
 */
void oracle_gemm_f64_block(int K, const uint8_t *A, int fmt_a, const uint8_t *B, int fmt_b,
                           double *C64, double *S, int m0, int m1, int n0, int n1)
{
    double ta[256], tb[256];
    oracle_fp8_decode_table(fmt_a, ta);
    oracle_fp8_decode_table(fmt_b, tb);
    const int nn = n1 - n0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int m = m0; m < m1; ++m) {
        double *arow = (double *)malloc(sizeof(double) * (size_t)K);
        const uint8_t *a = A + (int64_t)m * K;
        for (int k = 0; k < K; ++k) arow[k] = ta[a[k]];
        for (int n = n0; n < n1; ++n) {
            const uint8_t *b = B + (int64_t)n * K;
            double acc0 = 0, acc1 = 0, abs0 = 0, abs1 = 0;
            int k = 0;
            for (; k + 1 < K; k += 2) {
                double p0 = arow[k] * tb[b[k]];
                double p1 = arow[k + 1] * tb[b[k + 1]];
                acc0 += p0;
                acc1 += p1;
                abs0 += fabs(p0);
                abs1 += fabs(p1);
            }
            if (k < K) {
                double p0 = arow[k] * tb[b[k]];
                acc0 += p0;
                abs0 += fabs(p0);
            }
            C64[(int64_t)(m - m0) * nn + (n - n0)] = acc0 + acc1;
            S[(int64_t)(m - m0) * nn + (n - n0)] = abs0 + abs1;
        }
        free(arow);
    }
}

/* Same quantities for an arbitrary list of (m, n) coordinates. */
void oracle_gemm_f64_points(int K, const uint8_t *A, int fmt_a, const uint8_t *B, int fmt_b,
                            const int32_t *ms, const int32_t *ns, int64_t count,
                            double *C64, double *S)
{
    double ta[256], tb[256];
    oracle_fp8_decode_table(fmt_a, ta);
    oracle_fp8_decode_table(fmt_b, tb);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        const uint8_t *a = A + (int64_t)ms[i] * K;
        const uint8_t *b = B + (int64_t)ns[i] * K;
        double acc = 0, ab = 0;
        for (int k = 0; k < K; ++k) {
            double p = ta[a[k]] * tb[b[k]];
            acc += p;
            ab += fabs(p);
        }
        C64[i] = acc;
        S[i] = ab;
    }
}

/*
 * The acceptance rule: |C - C_ref| <= rel * S + abs_tol per element, with
 * rel = 1e-3 and abs_tol = 1e-6 for this path.  Returns the number of
 * elements that violate it; *worst receives the largest ratio
 * |C - C_ref| / (rel * S + abs_tol) seen (<= 1 means pass), *worst_index its
 * position.  NaN in C counts as a violation.
 */
int64_t oracle_check_tolerance(const float *C, const double *C64, const double *S,
                               int64_t count, double rel, double abs_tol,
                               double *worst, int64_t *worst_index)
{
    int64_t bad = 0;
    double w = 0.0;
    int64_t wi = -1;
    for (int64_t i = 0; i < count; ++i) {
        double err = fabs((double)C[i] - C64[i]);
        double lim = rel * S[i] + abs_tol;
        double ratio = err / lim;
        if (!(ratio <= 1.0)) ++bad;
        if (!(ratio <= w)) {
            w = isnan(ratio) ? INFINITY : ratio;
            wi = i;
        }
    }
    if (worst) *worst = w;
    if (worst_index) *worst_index = wi;
    return bad;
}

int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
