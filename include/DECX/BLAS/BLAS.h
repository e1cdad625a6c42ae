// Dense matrix multiplication on the GPU.  Signatures as in srcs/includes/DECX/BLAS/BLAS.h:67-81.
//
//   dst(M x N) = A(M x K) . B(K x N)                         plain
//   dst        = alpha . A . B + beta . C                    fused
//
// Matrices are created as (type, width, height): A = (t, K, M), B = (t, N, K), dst = (t, N, M).
// Types: de::_FP32_ (3xTF32 tensor-core path, fp32 accuracy), de::_FP16_ (fp32 accumulate, fp16 result),
// de::_COMPLEX_F32_ (interleaved {re, im}), de::_FP64_ and de::_COMPLEX_F64_ (fp64 tensor path).
// All operands and scalars must share one type.
// The calls are synchronous and return void; errors are written to *de::GetLastError():
// DECX_FAIL_DimsNotMatching (A.Width != B.Height, or C not M x N), DECX_FAIL_TYPE_MOT_MATCH,
// DECX_FAIL_UNSUPPORTED_TYPE, DECX_FAIL_CUDA_not_init, DECX_FAIL_CUDA_ALLOCATION, DECX_FAIL_CUDA_STREAM.
// dst is re-shaped (grow-only re-allocation) to N x M of A's type.
#ifndef DECX_B200_PUBLIC_BLAS_H_
#define DECX_B200_PUBLIC_BLAS_H_

#include "../classes/Matrix.h"
#include "../classes/GPU_Matrix.h"
#include "../classes/Vector.h"
#include "../classes/GPU_Vector.h"
#include "../classes/DecxNumber.h"

namespace de {
namespace cuda {
// dst (re-shaped to src.Height() x src.Width() columns x rows, i.e. width = src.Height()) = transpose of src; any
// element size of 1, 2, 4, 8 or 16 bytes.  Synchronous.  (srcs/includes/DECX/BLAS/BLAS.h:38,
// srcs/modules/BLAS/Basic_process/transpose/transpose.cu:50-101)
_DECX_API_ de::DH Transpose(de::GPU_Matrix& src, de::GPU_Matrix& dst);
}  // namespace cuda

// accumulation levels of the fp16 matrix-vector products (srcs/includes/DECX/classes/class_utils.h:126-140)
enum Fp16_Accuracy_Levels {
    Fp16_Accurate_L1 = 0,    // fp32 arithmetic, fp32 result vector
    Fp16_Accurate_L2 = 1,    // fp32 arithmetic, fp16 result
    Fp16_Accurate_L3 = 2     // fp16 arithmetic throughout, fp16 result: the caller minds overflow
};

namespace blas {
namespace cuda {
// device matrices (reference definitions: srcs/modules/BLAS/GEMM/CUDA/GEMM_LS.cu:315-393)
_DECX_API_ void GEMM(de::GPU_Matrix& A, de::GPU_Matrix& B, de::GPU_Matrix& dst);
_DECX_API_ void GEMM(de::GPU_Matrix& A, de::GPU_Matrix& B, de::GPU_Matrix& C, de::GPU_Matrix& dst,
                     const de::Number alpha, const de::Number beta);

// host matrices: declared by the reference (BLAS.h:69-70) but never defined there.  Here they copy,
// multiply and copy back in one pipelined pass; the 4-argument form computes dst = A.B + C.
_DECX_API_ void GEMM(de::Matrix& A, de::Matrix& B, de::Matrix& dst);
_DECX_API_ void GEMM(de::Matrix& A, de::Matrix& B, de::Matrix& C, de::Matrix& dst);

// Vector x Matrix and Matrix x Vector on host objects (srcs/includes/DECX/BLAS/BLAS.h:79-80, drivers
// srcs/modules/BLAS/GEMM/CUDA/VMM.cu:142-184): operands are copied to the device, multiplied in one pass over
// the matrix, and the result is copied back.  fp32, or fp16 with the accumulation level `_fp16_accu`
// (dst is an fp32 vector for Fp16_Accurate_L1, fp16 otherwise).  dst is re-shaped.  Errors through
// de::GetLastError(), which these two reset on entry like the reference.
//   dst[j] = sum_k A[k] * B(k, j)      A.Len() == B.Height(),  dst.Len() = B.Width()
_DECX_API_ void GEMM(de::Vector& A, de::Matrix& B, de::Vector& dst, const uint32_t _fp16_accu = 0);
//   dst[i] = sum_k A(i, k) * B[k]      A.Width() == B.Len(),   dst.Len() = A.Height()
_DECX_API_ void GEMM(de::Matrix& A, de::Vector& B, de::Vector& dst, const uint32_t _fp16_accu = 0);
}  // namespace cuda
}  // namespace blas
}  // namespace de
#endif
