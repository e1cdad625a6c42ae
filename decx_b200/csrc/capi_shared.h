// Small internals shared by the translation units of libdecx_b200.so.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace dxb_host {

// per-thread count of kernels launched by the current C-ABI call (decxb200_last_launch_count)
void count_launch(int n = 1);
void reset_launches();

inline uint64_t round_up(uint64_t x, uint64_t m) { return (x + m - 1) / m * m; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// fp64 / complex-fp64 GEMM on `stream` (real expansion of B in `workspace` for the complex case;
// b_expanded: the workspace already holds it, e.g. from the previous row block of the same B)
int run_f64(cudaStream_t stream, bool cplx, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda,
            const void* B, uint64_t ldb, const void* C, uint64_t ldc, void* D, uint64_t ldd, const double alpha[2],
            const double beta[2], void* workspace, size_t workspace_bytes, bool b_expanded = false);
size_t f64_workspace_bytes(bool cplx, uint32_t M, uint32_t N, uint32_t K);

// D = A . B in 3xTF32 from operands that a producer kernel already wrote as tf32 (hi, lo) planes: rows ldaw / ldbw
// floats apart (multiples of 32), planes 256-byte aligned; the planes' padding columns need not be initialised.
int gemm_tf32_planes(cudaStream_t stream, uint32_t M, uint32_t N, uint32_t K, const float* a_hi, const float* a_lo,
                     uint64_t ldaw, const float* b_hi, const float* b_lo, uint64_t ldbw, void* D, uint64_t ldd,
                     unsigned* status);

// fp32 convolution as an implicit GEMM: the kernel's operand tiles are TMA boxes of the zero-bordered source planes.
struct ConvPlanes {
    const float *src_hi, *src_lo;     // Hp x Wp x Cp each (Cp % 4 == 0), Hp >= (OH-1)*sy + kh, Wp >= (OW-1)*sx + kw
    uint32_t Wp, Cp;
    const float *b_hi, *b_lo;         // (kh * round_up(kw*Cp, 32)) x n, rows ldbw floats apart
    uint64_t ldbw;
    uint32_t kh, kw, n, sx, sy, OH, OW;
    float* dst;                       // OH x OW x n, 16-byte aligned, dst_dpitch % 4 == 0, n % 4 == 0
    uint32_t dst_wpitch, dst_dpitch;
    uint32_t tw;                      // output positions of one tile row: 32, 64 or 128
};
int conv_tf32_implicit(cudaStream_t stream, const ConvPlanes& c, unsigned* status);

}  // namespace dxb_host
