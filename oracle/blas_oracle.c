/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the matrix-vector products, of the fp64 GEMMs and of the fp32
 * 2-D convolution (parity unpinned for the convolution, see its function).
 * Only tests, the smoke check and the benchmark's cpu_baseline leg may call this file.
 *
 * What it restates (reference, file:line within param0037/DECX):
 *   y[i] = sum_k A[i][k] x[k]   (Matrix x Vector)  srcs/modules/BLAS/GEMM/CUDA/extreme_shapes/VMM_fp32.cu (cu_mat_m_vec_fp32),
 *   y[j] = sum_k x[k] A[k][j]   (Vector x Matrix)  VMM_fp32.cu (cu_vec_m_mat_fp32), fp16 forms VMM_fp16.cu:35-424;
 *                                                  drivers srcs/modules/BLAS/GEMM/CUDA/VMM.cu:55-184
 *   dst = alpha * A * B + beta * C in fp64 / complex fp64
 *                                                  srcs/modules/BLAS/GEMM/CUDA/large_squares/GEMM_kernels.cuh:31-62,
 *                                                  64b/GEMM_fp64_B64_kernels.cu:58, cplxd/GEMM_cplxd_B64_kernels.cu:60
 * Precision: fp32 vectors are accumulated in fp64; fp16 products (exact in fp32) are accumulated in fp32 in
 * index order for the fp32-arithmetic levels and in fp64 for the bound the fp16-arithmetic level is held to;
 * fp64 problems are accumulated in long double (64-bit significand on x86-64).
 * Pinning: the fp64 GEMM restatement is checked against outputs of the reference's own de::blas::cpu::GEMM
 * (fp64 case, srcs/modules/BLAS/GEMM/CPU/GEMM.cxx:50-113) where that build exists, and against numpy; the
 * reference holds no known-answer vectors for the matrix-vector products (parity unpinned for those beyond
 * numpy's own dot product).
 */
#include <stddef.h>
#include <stdint.h>

#define ORACLE_API __attribute__((visibility("default")))

static float h2f(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    union { uint32_t u; float f; } c;
    c.u = bits;
    return c.f;
}

/* trans == 0: y[rows] = A x[cols]; trans == 1: y[cols] = x[rows] A.  A is rows x cols, lda elements per row. */
ORACLE_API void oracle_gemv_f32(int trans, uint32_t rows, uint32_t cols, const float* A, size_t lda, const float* x,
                                double* y) {
    if (!trans) {
        for (uint32_t i = 0; i < rows; ++i) {
            double s = 0.0;
            for (uint32_t k = 0; k < cols; ++k) s += (double)A[i * lda + k] * (double)x[k];
            y[i] = s;
        }
    } else {
        for (uint32_t j = 0; j < cols; ++j) y[j] = 0.0;
        for (uint32_t k = 0; k < rows; ++k) {
            const double xk = x[k];
            for (uint32_t j = 0; j < cols; ++j) y[j] += xk * (double)A[k * lda + j];
        }
    }
}

/* fp16 inputs: y32 = fp32 accumulation in index order, y64 = fp64 accumulation, mag = sum |a||x| (error scale) */
ORACLE_API void oracle_gemv_f16(int trans, uint32_t rows, uint32_t cols, const uint16_t* A, size_t lda,
                                const uint16_t* x, float* y32, double* y64, double* mag) {
    const uint32_t n = trans ? cols : rows, red = trans ? rows : cols;
    for (uint32_t o = 0; o < n; ++o) {
        float s = 0.f;
        double d = 0.0, m = 0.0;
        for (uint32_t k = 0; k < red; ++k) {
            const float a = trans ? h2f(A[k * lda + o]) : h2f(A[o * lda + k]);
            const float p = a * h2f(x[k]);                /* exact: 11-bit x 11-bit significands */
            s += p;
            d += (double)p;
            m += p < 0 ? -(double)p : (double)p;
        }
        y32[o] = s;
        y64[o] = d;
        mag[o] = m;
    }
}

/* D = alpha A B + beta C in fp64 with long double accumulation; C may be NULL */
ORACLE_API void oracle_gemm_f64(uint32_t M, uint32_t N, uint32_t K, const double* A, size_t lda, const double* B,
                                size_t ldb, const double* C, size_t ldc, double alpha, double beta, double* D,
                                size_t ldd) {
    for (uint32_t i = 0; i < M; ++i)
        for (uint32_t j = 0; j < N; ++j) {
            long double s = 0.0L;
            for (uint32_t k = 0; k < K; ++k) s += (long double)A[i * lda + k] * (long double)B[k * ldb + j];
            s *= (long double)alpha;
            if (C) s += (long double)beta * (long double)C[i * ldc + j];
            D[i * ldd + j] = (double)s;
        }
}

/* complex: interleaved (re, im) doubles; pitches in complex elements; alpha, beta = {re, im} */
ORACLE_API void oracle_gemm_c64(uint32_t M, uint32_t N, uint32_t K, const double* A, size_t lda, const double* B,
                                size_t ldb, const double* C, size_t ldc, const double* alpha, const double* beta,
                                double* D, size_t ldd) {
    for (uint32_t i = 0; i < M; ++i)
        for (uint32_t j = 0; j < N; ++j) {
            long double re = 0.0L, im = 0.0L;
            for (uint32_t k = 0; k < K; ++k) {
                const long double ar = A[2 * (i * lda + k)], ai = A[2 * (i * lda + k) + 1];
                const long double br = B[2 * (k * ldb + j)], bi = B[2 * (k * ldb + j) + 1];
                re += ar * br - ai * bi;
                im += ar * bi + ai * br;
            }
            long double ore = alpha[0] * re - alpha[1] * im, oim = alpha[0] * im + alpha[1] * re;
            if (C) {
                const long double cr = C[2 * (i * ldc + j)], ci = C[2 * (i * ldc + j) + 1];
                ore += beta[0] * cr - beta[1] * ci;
                oim += beta[0] * ci + beta[1] * cr;
            }
            D[2 * (i * ldd + j)] = (double)ore;
            D[2 * (i * ldd + j) + 1] = (double)oim;
        }
}

/* Direct 2-D cross-correlation, fp64 accumulation (reference: de::nn::cuda::Conv2D, srcs/modules/NN/convolution/CUDA/
 * fp32/Conv2D.cu:57-131; output dims cuda_conv2D_fp32_im2col_planner.cu:215-225; zero border of kh/2, kw/2 and the
 * bottom bound OH*sy of im2col_fp32.cu:122-132).  Dense tensors: src H x W x C, kernels n x kh x kw x C,
 * dst OH x OW x n; mag = sum |src||kernel| per output (error scale).  extend: 0 none, 2 constant.
 * PARITY UNPINNED: the reference has no CPU Conv2D, test or golden vector; this follows a reading of its CUDA path and
 * is cross-checked against an independent numpy formulation only. */
ORACLE_API int oracle_conv2d_f32(uint32_t H, uint32_t W, uint32_t C, const float* src, uint32_t kh, uint32_t kw, uint32_t n,
                                 const float* ker, uint32_t sx, uint32_t sy, int extend, uint32_t OH, uint32_t OW, double* dst,
                                 double* mag) {
    uint32_t eh, ew, py = 0, px = 0, hlim = H;
    if (extend == 0) {
        if (kh > H || kw > W) return -1;
        eh = (H - kh + 1) / sy;
        ew = (W - kw + 1) / sx;
    } else if (extend == 2) {
        eh = H / sy;
        ew = W / sx;
        py = kh / 2;
        px = kw / 2;
        hlim = eh * sy;
    } else {
        return -1;
    }
    if (eh != OH || ew != OW) return -2;
    for (uint32_t y = 0; y < OH; ++y)
        for (uint32_t x = 0; x < OW; ++x)
            for (uint32_t t = 0; t < n; ++t) {
                double s = 0.0, m = 0.0;
                for (uint32_t i = 0; i < kh; ++i) {
                    const int64_t yy = (int64_t)y * sy + i - py;
                    if (yy < 0 || yy >= (int64_t)hlim) continue;
                    for (uint32_t j = 0; j < kw; ++j) {
                        const int64_t xx = (int64_t)x * sx + j - px;
                        if (xx < 0 || xx >= (int64_t)W) continue;
                        const float* a = src + ((size_t)yy * W + (size_t)xx) * C;
                        const float* b = ker + (((size_t)t * kh + i) * kw + j) * C;
                        for (uint32_t c = 0; c < C; ++c) {
                            const double p = (double)a[c] * (double)b[c];
                            s += p;
                            m += p < 0 ? -p : p;
                        }
                    }
                }
                dst[((size_t)y * OW + x) * n + t] = s;
                mag[((size_t)y * OW + x) * n + t] = m;
            }
    return 0;
}
