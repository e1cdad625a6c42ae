// fp64 and complex-fp64 GEMM:  D = alpha * A * B + beta * C, row-major, pitched
// (reference: the _FP64_ / _COMPLEX_F64_ cases of de::blas::cuda::GEMM, srcs/modules/BLAS/GEMM/CUDA/GEMM_LS.cu:335-345,
// SIMT kernels large_squares/64b/GEMM_fp64_B64_kernels.cu:58 and cplxd/GEMM_cplxd_B64_kernels.cu:60).
//
// tcgen05 has no fp64 kind, so the fp64 tensor path of this chip is the warp-level DMMA
// (mma.sync.m8n8k4.f64).  CTA tile 128 x 128 x 16, eight warps as 2 x 4, each warp a 64 x 32 tile = 8 x 4
// DMMA tiles accumulated in registers; operands reach shared memory through a three-stage cp.async ring
// (16-byte copies, zero fill outside the matrix, so ragged M / N / K need no padding); rows of the shared tiles
// are padded so that the fragment loads of a half-warp hit 16 different 8-byte banks.
// A complex problem arrives here as the real problem of twice the K and N extents (A viewed as M x 2K reals,
// B expanded by expand_cplxd_b_kernel); only the epilogue knows about (re, im) pairs -- the two accumulator
// elements a thread holds per DMMA tile are exactly one complex number.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace dxb {

#ifndef DXB_F64_BK
#define DXB_F64_BK 16
#endif
constexpr int F64_BM = 128, F64_BN = 128, F64_BK = DXB_F64_BK, F64_STAGES = 3, F64_THREADS = 256;
constexpr int F64_LDA_S = F64_BK + 4;       // 20 doubles per row of the A tile
constexpr int F64_LDB_S = F64_BN + 4;       // 132 doubles per row of the B tile
constexpr int F64_A_STAGE = F64_BM * F64_LDA_S;
constexpr int F64_B_STAGE = F64_BK * F64_LDB_S;
constexpr int F64_SMEM_BYTES = F64_STAGES * (F64_A_STAGE + F64_B_STAGE) * 8;

struct GemmF64Params {
    const double* A; const double* B; const double* C; double* D;
    uint64_t lda, ldb, ldc, ldd;            // in doubles
    uint32_t M, N, K;                       // real extents (complex: N, K doubled)
    double alpha_re, alpha_im, beta_re, beta_im;
    int complex_epilogue;
    int vec_a, vec_b;                       // 16-byte copies legal for A / B (base and pitch aligned)
    uint32_t tiles_n, group_m;
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void dmma_8x8x4(double (&c)[2], double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
                 : "+d"(c[0]), "+d"(c[1]) : "d"(a), "d"(b));
}

// one pair of doubles at (row, col..col+1) of a rows x cols matrix -> shared; zero outside
__device__ __forceinline__ void load_pair(uint32_t dst, const double* base, uint64_t ld, uint32_t row, uint32_t col,
                                          uint32_t rows, uint32_t cols, int vec) {
    const bool in_row = row < rows;
    const uint32_t n = (in_row && col < cols) ? (col + 1 < cols ? 2u : 1u) : 0u;
    // the source address must stay valid even when nothing is read from it
    const double* src = base + (in_row ? uint64_t(row) * ld : 0) + (n ? col : 0);
    if (vec) {
        cp_async_16(dst, n ? src : base, n * 8);
    } else {
        cp_async_8(dst, n ? src : base, n ? 8u : 0u);
        cp_async_8(dst + 8, n == 2 ? src + 1 : base, n == 2 ? 8u : 0u);
    }
}

__global__ void __launch_bounds__(F64_THREADS, 1) gemm_f64_kernel(const GemmF64Params p) {
    extern __shared__ __align__(16) uint8_t f64_smem[];
    double* As = reinterpret_cast<double*>(f64_smem);
    double* Bs = As + F64_STAGES * F64_A_STAGE;
    const uint32_t as_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(As));
    const uint32_t bs_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(Bs));

    // tile of this CTA: groups of `group_m` tile rows walked column by column (L2 reuse of the A rows)
    const uint32_t t = blockIdx.x;
    const uint32_t tiles_m = (p.M + F64_BM - 1) / F64_BM;
    const uint32_t per_group = p.group_m * p.tiles_n;
    const uint32_t g = t / per_group, first_m = g * p.group_m;
    const uint32_t rows_g = min(p.group_m, tiles_m - first_m);
    const uint32_t r = t - g * per_group;
    const uint32_t m0 = (first_m + r % rows_g) * F64_BM, n0 = (r / rows_g) * F64_BN;

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t wm = warp >> 2, wn = warp & 3;           // 2 x 4 warps
    const uint32_t gid = lane >> 2, q = lane & 3;

    double acc[8][4][2];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    const uint32_t n_kt = (p.K + F64_BK - 1) / F64_BK;
    auto issue = [&](uint32_t kt, uint32_t stage) {
        const uint32_t k0 = kt * F64_BK;
        // A tile: 128 rows x BK/2 pairs; B tile: BK rows x 64 pairs; 64 * BK pairs each, BK/4 per thread
        constexpr uint32_t APR = F64_BK / 2;                // pairs per row of the A tile
#pragma unroll
        for (int i = 0; i < F64_BK / 4; ++i) {
            const uint32_t c = tid + i * F64_THREADS;
            const uint32_t ar = c / APR, ap = (c % APR) * 2;
            load_pair(as_u32 + (stage * F64_A_STAGE + ar * F64_LDA_S + ap) * 8, p.A, p.lda, m0 + ar, k0 + ap, p.M, p.K,
                      p.vec_a);
            const uint32_t br = c >> 6, bp = (c & 63) * 2;
            load_pair(bs_u32 + (stage * F64_B_STAGE + br * F64_LDB_S + bp) * 8, p.B, p.ldb, k0 + br, n0 + bp, p.K, p.N,
                      p.vec_b);
        }
    };
#pragma unroll
    for (int s = 0; s < F64_STAGES - 1; ++s) {
        if (uint32_t(s) < n_kt) issue(s, s);
        cp_async_commit();
    }
    for (uint32_t kt = 0; kt < n_kt; ++kt) {
        cp_async_wait<F64_STAGES - 2>();
        __syncthreads();                                    // stage kt is complete; stage kt-1 is free for refill
        const uint32_t nk = kt + F64_STAGES - 1;
        if (nk < n_kt) issue(nk, nk % F64_STAGES);
        cp_async_commit();
        const double* a_s = As + (kt % F64_STAGES) * F64_A_STAGE + (wm * 64 + gid) * F64_LDA_S + q;
        const double* b_s = Bs + (kt % F64_STAGES) * F64_B_STAGE + q * F64_LDB_S + wn * 32 + gid;
#pragma unroll
        for (int kk = 0; kk < F64_BK / 4; ++kk) {
            double a[8], b[4];
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = a_s[i * 8 * F64_LDA_S + kk * 4];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = b_s[kk * 4 * F64_LDB_S + j * 8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) dmma_8x8x4(acc[i][j], a[i], b[j]);
        }
    }
    cp_async_wait<0>();

    // epilogue: a thread holds columns (2q, 2q+1) of row gid of every 8 x 8 tile
    const bool has_c = p.C != nullptr;
    const bool vec_d = ((p.ldd & 1) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0);
    const bool vec_c = has_c && ((p.ldc & 1) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t row = m0 + wm * 64 + i * 8 + gid;
        if (row >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t col = n0 + wn * 32 + j * 8 + q * 2;
            if (col >= p.N) continue;
            const bool two = col + 1 < p.N;
            double v0 = acc[i][j][0], v1 = acc[i][j][1], c0 = 0.0, c1 = 0.0;
            if (has_c) {
                const double* cp = p.C + uint64_t(row) * p.ldc + col;
                if (two && vec_c) { const double2 cc = *reinterpret_cast<const double2*>(cp); c0 = cc.x; c1 = cc.y; }
                else { c0 = cp[0]; if (two) c1 = cp[1]; }
            }
            if (p.complex_epilogue) {                       // (v0, v1) = (re, im); N is even here
                const double re = p.alpha_re * v0 - p.alpha_im * v1 + p.beta_re * c0 - p.beta_im * c1;
                const double im = p.alpha_re * v1 + p.alpha_im * v0 + p.beta_re * c1 + p.beta_im * c0;
                v0 = re; v1 = im;
            } else {
                v0 = p.alpha_re * v0 + p.beta_re * c0;
                v1 = p.alpha_re * v1 + p.beta_re * c1;
            }
            double* dp = p.D + uint64_t(row) * p.ldd + col;
            if (two && vec_d) *reinterpret_cast<double2*>(dp) = make_double2(v0, v1);
            else { dp[0] = v0; if (two) dp[1] = v1; }
        }
    }
}

// B: K x N complex doubles (ldb complex elements per row) -> its 2K x 2N real expansion (ldw doubles per row):
// row 2k = (re, im) pairs of row k, row 2k+1 = (-im, re) pairs, so that A (viewed as M x 2K reals) times it is
// the complex product in interleaved storage (the 4-real-multiplication form of
// srcs/modules/BLAS/GEMM/CUDA/large_squares/cplxd/GEMM_cplxd_B64_kernels.cu:60).
__global__ void expand_cplxd_b_kernel(const double2* __restrict__ B, uint64_t ldb, uint32_t K, uint32_t N,
                                      double* __restrict__ W, uint64_t ldw) {
    const uint64_t total = uint64_t(K) * N;
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t k = uint32_t(i / N), n = uint32_t(i % N);
        const double2 b = B[uint64_t(k) * ldb + n];
        *reinterpret_cast<double2*>(W + uint64_t(2 * k) * ldw + 2 * n) = make_double2(b.x, b.y);
        *reinterpret_cast<double2*>(W + uint64_t(2 * k + 1) * ldw + 2 * n) = make_double2(-b.y, b.x);
    }
}

}  // namespace dxb
