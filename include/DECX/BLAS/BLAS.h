// Dense matrix multiplication on the GPU.  Signatures as in srcs/includes/DECX/BLAS/BLAS.h:67-81.
//
//   dst(M x N) = A(M x K) . B(K x N)                         plain
//   dst        = alpha . A . B + beta . C                    fused
//
// Matrices are created as (type, width, height): A = (t, K, M), B = (t, N, K), dst = (t, N, M).
// Types: de::_FP32_ (3xTF32 tensor-core path, fp32 accuracy), de::_FP16_ (fp32 accumulate, fp16 result),
// de::_COMPLEX_F32_ (interleaved {re, im}).  All operands and scalars must share one type.
// The calls are synchronous and return void; errors are written to *de::GetLastError():
// DECX_FAIL_DimsNotMatching (A.Width != B.Height, or C not M x N), DECX_FAIL_TYPE_MOT_MATCH,
// DECX_FAIL_UNSUPPORTED_TYPE, DECX_FAIL_CUDA_not_init, DECX_FAIL_CUDA_ALLOCATION, DECX_FAIL_CUDA_STREAM.
// dst is re-shaped (grow-only re-allocation) to N x M of A's type.
#ifndef DECX_B200_PUBLIC_BLAS_H_
#define DECX_B200_PUBLIC_BLAS_H_

#include "../classes/Matrix.h"
#include "../classes/GPU_Matrix.h"
#include "../classes/DecxNumber.h"

namespace de {
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
}  // namespace cuda
}  // namespace blas
}  // namespace de
#endif
