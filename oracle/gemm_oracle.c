/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the arithmetic of DECX's dense GEMM.
 *
 * Only tests, the smoke check and the benchmark's cpu_baseline leg may call this file.
 * The product path (decx_b200/) never links, imports or executes it.
 *
 * What it restates (reference, file:line within param0037/DECX):
 *   dst = A * B                    srcs/modules/BLAS/GEMM/CUDA/large_squares/GEMM_kernels.cuh:31-50
 *   dst = alpha * A * B + beta * C srcs/modules/BLAS/GEMM/CUDA/large_squares/GEMM_kernels.cuh:53-62
 *                                  (e.g. fp32/GEMM_fp32_B128_kernels.cu:723-748)
 *   complex multiply-accumulate    srcs/modules/BLAS/GEMM/CUDA/large_squares/64b/GEMM_cplxf_B64_kernels.cu:35-44
 *   row-major pitched addressing   srcs/includes/DECX/classes/Matrix.h:64-68 (base + pitch*row + col)
 * Where the reference kernels deviate from this formula on the fused path (they read dst
 * instead of C, apply alpha twice for complex, fold beta*C into an fp16 partial sum), the
 * formula above is what is restated, not the deviation.
 *
 * Precision follows the parity contract of this path: fp32 and complex-fp32 inputs are
 * multiplied and accumulated in fp64; fp16 inputs are accumulated in fp32 (products of two
 * halves are exact in fp32) and the result is left in fp32 (the caller rounds to half when
 * it wants the stored value).
 *
 * Pinning: checked against (1) the closed-form answer of the reference's only GEMM
 * known-answer program, samples/Matrix_Multiplication/MatMul.cpp:64-140
 * (A[i][j] = j, B[i][j] = i, C = (1e6, 1e6) -> (sum_{i<K} i^2 + 1e6, 1e6)), and (2) the
 * outputs of the reference's own de::blas::cpu::GEMM built from its sources into
 * oracle/_ref/ (tests/test_oracle.py; stored outputs in tests/golden/).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ---- row-parallel helper (plain pthreads; the image has no OpenMP runtime) ---- */
typedef void (*row_fn)(int64_t row, void* ctx);
typedef struct { row_fn fn; void* ctx; int64_t rows; volatile int64_t* next; } par_job;
static int g_threads = 0; /* 0 = number of online CPUs */
ORACLE_API void oracle_set_threads(int n) { g_threads = n; }
static void* par_worker(void* arg) {
    par_job* j = (par_job*)arg;
    for (;;) {
        const int64_t r0 = __sync_fetch_and_add(j->next, 4);
        if (r0 >= j->rows) break;
        const int64_t r1 = (r0 + 4 < j->rows) ? r0 + 4 : j->rows;
        for (int64_t r = r0; r < r1; ++r) j->fn(r, j->ctx);
    }
    return NULL;
}
static void par_rows(int64_t rows, row_fn fn, void* ctx) {
    long n = g_threads > 0 ? g_threads : sysconf(_SC_NPROCESSORS_ONLN);
    if (n < 1) n = 1;
    if (n > 64) n = 64;
    if (n > rows) n = rows > 0 ? rows : 1;
    volatile int64_t next = 0;
    par_job job = {fn, ctx, rows, &next};
    pthread_t th[64];
    int started = 0;
    for (long t = 1; t < n; ++t)
        if (pthread_create(&th[started], NULL, par_worker, &job) == 0) ++started;
    par_worker(&job);
    for (int t = 0; t < started; ++t) pthread_join(th[t], NULL);
}

/* IEEE binary16 -> binary32, exact. */
static float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
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

/* binary32 -> binary16, round to nearest even (the rounding of the fp16 GEMM's final store). */
static uint16_t float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | ((x > 0x7F800000u) ? 0x200u : 0u));
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);           /* rounds to inf */
    if (x < 0x33000001u) return (uint16_t)sign;                         /* rounds to zero */
    int32_t e = (int32_t)(x >> 23) - 127;
    uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t hexp;
    if (e < -14) { shift = 13 + (-14 - e); hexp = 0; } else { shift = 13; hexp = (uint32_t)(e + 15); }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    if (hexp == 0) return (uint16_t)(sign | q);                         /* q may carry into exp 1: still right */
    return (uint16_t)(sign | (((hexp - 1) << 10) + q));                 /* q carries the hidden bit */
}

ORACLE_API void oracle_half_to_float(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = half_to_float(src[i]);
}
ORACLE_API void oracle_float_to_half(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = float_to_half(src[i]);
}

typedef struct {
    uint32_t M, N, K; const float* A; size_t lda; const float* B; size_t ldb; const float* C; size_t ldc;
    double alpha, beta; double* D; size_t ldd;
} f32_ctx;
static void f32_row(int64_t i, void* p) {
    const f32_ctx* c = (const f32_ctx*)p;
    double* acc = c->D + (size_t)i * c->ldd;
    for (uint32_t j = 0; j < c->N; ++j) acc[j] = 0.0;
    for (uint32_t k = 0; k < c->K; ++k) {
        const double a = (double)c->A[(size_t)i * c->lda + k];
        const float* brow = c->B + (size_t)k * c->ldb;
        for (uint32_t j = 0; j < c->N; ++j) acc[j] += a * (double)brow[j];
    }
    for (uint32_t j = 0; j < c->N; ++j) {
        double v = c->alpha * acc[j];
        if (c->C != NULL) v += c->beta * (double)c->C[(size_t)i * c->ldc + j];
        acc[j] = v;
    }
}

/*
 * fp32 inputs, fp64 arithmetic:  D = alpha * A*B + beta * C   (C may be NULL -> beta ignored)
 * A: M x K (lda), B: K x N (ldb), C: M x N (ldc), D: M x N doubles (ldd).
 */
ORACLE_API void oracle_gemm_f32(uint32_t M, uint32_t N, uint32_t K, const float* A, size_t lda, const float* B,
                                size_t ldb, const float* C, size_t ldc, double alpha, double beta, double* D,
                                size_t ldd) {
    f32_ctx c = {M, N, K, A, lda, B, ldb, C, ldc, alpha, beta, D, ldd};
    par_rows((int64_t)M, f32_row, &c);
}

typedef struct {
    uint32_t M, N, K; const float* A; size_t lda; const float* B; size_t ldb; const float* C; size_t ldc;
    double alpha[2], beta[2]; double* D; size_t ldd;
} c32_ctx;
static void c32_row(int64_t i, void* p) {
    const c32_ctx* c = (const c32_ctx*)p;
    double* acc = c->D + 2 * (size_t)i * c->ldd;
    for (uint32_t j = 0; j < 2 * c->N; ++j) acc[j] = 0.0;
    for (uint32_t k = 0; k < c->K; ++k) {
        const double ar = (double)c->A[2 * ((size_t)i * c->lda + k)];
        const double ai = (double)c->A[2 * ((size_t)i * c->lda + k) + 1];
        const float* brow = c->B + 2 * (size_t)k * c->ldb;
        for (uint32_t j = 0; j < c->N; ++j) {
            const double br = (double)brow[2 * j], bi = (double)brow[2 * j + 1];
            acc[2 * j] += ar * br - ai * bi;      /* real part      */
            acc[2 * j + 1] += ar * bi + ai * br;  /* imaginary part */
        }
    }
    for (uint32_t j = 0; j < c->N; ++j) {
        const double re = acc[2 * j], im = acc[2 * j + 1];
        double ore = c->alpha[0] * re - c->alpha[1] * im;
        double oim = c->alpha[0] * im + c->alpha[1] * re;
        if (c->C != NULL) {
            const double cr = (double)c->C[2 * ((size_t)i * c->ldc + j)];
            const double ci = (double)c->C[2 * ((size_t)i * c->ldc + j) + 1];
            ore += c->beta[0] * cr - c->beta[1] * ci;
            oim += c->beta[0] * ci + c->beta[1] * cr;
        }
        acc[2 * j] = ore;
        acc[2 * j + 1] = oim;
    }
}

/*
 * interleaved complex fp32 inputs {re, im}, fp64 arithmetic.  ld* count complex elements.
 * alpha, beta: {re, im}.  D: M x N complex doubles, interleaved.
 */
ORACLE_API void oracle_gemm_c32(uint32_t M, uint32_t N, uint32_t K, const float* A, size_t lda, const float* B,
                                size_t ldb, const float* C, size_t ldc, const double* alpha, const double* beta,
                                double* D, size_t ldd) {
    c32_ctx c = {M, N, K, A, lda, B, ldb, C, ldc, {alpha[0], alpha[1]}, {0.0, 0.0}, D, ldd};
    if (beta != NULL) { c.beta[0] = beta[0]; c.beta[1] = beta[1]; }
    par_rows((int64_t)M, c32_row, &c);
}

typedef struct {
    uint32_t M, N, K; const uint16_t* A; size_t lda; const float* Bf; const uint16_t* C; size_t ldc;
    float alpha, beta; float* D; size_t ldd;
} f16_ctx;
static void f16_row(int64_t i, void* p) {
    const f16_ctx* c = (const f16_ctx*)p;
    float* acc = c->D + (size_t)i * c->ldd;
    for (uint32_t j = 0; j < c->N; ++j) acc[j] = 0.0f;
    for (uint32_t k = 0; k < c->K; ++k) {
        const float a = half_to_float(c->A[(size_t)i * c->lda + k]);
        const float* brow = c->Bf + (size_t)k * c->N;
        for (uint32_t j = 0; j < c->N; ++j) acc[j] += a * brow[j];
    }
    for (uint32_t j = 0; j < c->N; ++j) {
        float v = c->alpha * acc[j];
        if (c->C != NULL) v += c->beta * half_to_float(c->C[(size_t)i * c->ldc + j]);
        acc[j] = v;
    }
}

/*
 * fp16 inputs (raw binary16 words), fp32 accumulation in increasing k, fp32 result.
 */
ORACLE_API void oracle_gemm_f16(uint32_t M, uint32_t N, uint32_t K, const uint16_t* A, size_t lda, const uint16_t* B,
                                size_t ldb, const uint16_t* C, size_t ldc, float alpha, float beta, float* D,
                                size_t ldd) {
    float* Bf = (float*)malloc((size_t)K * N * sizeof(float));
    if (Bf == NULL) return;
    for (uint32_t k = 0; k < K; ++k)
        for (uint32_t j = 0; j < N; ++j) Bf[(size_t)k * N + j] = half_to_float(B[(size_t)k * ldb + j]);
    f16_ctx c = {M, N, K, A, lda, Bf, C, ldc, alpha, beta, D, ldd};
    par_rows((int64_t)M, f16_row, &c);
    free(Bf);
}

/*
 * Parity metric of this path:
 *     max_ij |D_ij - Dref_ij| / ( ||A_i,:||_2 * ||B_:,j||_2 )
 * `cplx` != 0: all arrays are interleaved complex and |.| is the complex modulus.
 * row_norm: M doubles, col_norm: N doubles (from oracle_norms_*).  Entries whose denominator
 * is zero are compared exactly (any difference yields +inf).  Returns the maximum, or NaN if
 * any compared entry is NaN.
 */
ORACLE_API double oracle_metric(uint32_t M, uint32_t N, int cplx, const double* D, size_t ldd, const double* Dref,
                                size_t ldr, const double* row_norm, const double* col_norm) {
    double worst = 0.0;
    for (uint32_t i = 0; i < M; ++i) {
        for (uint32_t j = 0; j < N; ++j) {
            double err;
            if (cplx) {
                const double dr = D[2 * ((size_t)i * ldd + j)] - Dref[2 * ((size_t)i * ldr + j)];
                const double di = D[2 * ((size_t)i * ldd + j) + 1] - Dref[2 * ((size_t)i * ldr + j) + 1];
                err = sqrt(dr * dr + di * di);
            } else {
                err = fabs(D[(size_t)i * ldd + j] - Dref[(size_t)i * ldr + j]);
            }
            const double den = row_norm[i] * col_norm[j];
            double m;
            if (den > 0.0) m = err / den;
            else m = (err == 0.0) ? 0.0 : INFINITY;
            if (m != m) return NAN;       /* a NaN anywhere in D or Dref fails the comparison */
            if (m > worst) worst = m;
        }
    }
    return worst;
}

/* 2-norms of the rows of A (M x K) and of the columns of B (K x N); `cplx`: interleaved complex floats. */
ORACLE_API void oracle_norms_f32(uint32_t M, uint32_t N, uint32_t K, int cplx, const float* A, size_t lda,
                                 const float* B, size_t ldb, double* row_norm, double* col_norm) {
    const uint32_t w = cplx ? 2u : 1u;
    for (uint32_t i = 0; i < M; ++i) {
        double s = 0.0;
        for (uint32_t k = 0; k < w * K; ++k) {
            const double v = (double)A[w * (size_t)i * lda + k];
            s += v * v;
        }
        row_norm[i] = sqrt(s);
    }
    for (uint32_t j = 0; j < N; ++j) col_norm[j] = 0.0;
    for (uint32_t k = 0; k < K; ++k)
        for (uint32_t j = 0; j < N; ++j)
            for (uint32_t c = 0; c < w; ++c) {
                const double v = (double)B[w * ((size_t)k * ldb + j) + c];
                col_norm[j] += v * v;
            }
    for (uint32_t j = 0; j < N; ++j) col_norm[j] = sqrt(col_norm[j]);
}
