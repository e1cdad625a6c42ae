// Element type casts of device matrices.  Method values as in srcs/includes/DECX/basic_proc/type_cast.h:22-42;
// de::cuda::TypeCast(GPU_Matrix&, GPU_Matrix&, int) is defined by the reference in
// srcs/modules/BLAS/Basic_process/type_cast/GPU_Matrix_type_cast.cu:38-85 (fp32<->fp64 and int32->fp32 work
// there).  CVT_FP32_FP16 / CVT_FP16_FP32 are new: the device-side way to make the operands of the fp16 GEMM
// (the reference can only convert element by element on the host, de::Float2Half).
#ifndef DECX_B200_PUBLIC_TYPE_CAST_H_
#define DECX_B200_PUBLIC_TYPE_CAST_H_

#include "../basic.h"
#include "../classes/GPU_Matrix.h"

namespace de {
enum TypeCast_Method {
    CVT_INT32_UINT8 = 0,
    CVT_UINT8_CLAMP_TO_ZERO = 1,
    CVT_INT32_UINT8_TRUNCATE = 2,
    CVT_FP32_FP64 = 4,
    CVT_UINT8_CYCLIC = 5,
    CVT_FP64_FP32 = 6,
    CVT_INT32_FP32 = 7,
    CVT_FP32_INT32 = 8,
    CVT_UINT8_SATURATED = 9,
    CVT_UINT8_INT32 = 10,
    CVT_FP32_UINT8 = 16,
    CVT_UINT8_FP32 = 17,
    CVT_FP32_FP16 = 32,      // round to nearest even (new)
    CVT_FP16_FP32 = 33       // exact (new)
};

namespace cuda {
// dst is re-shaped to src's extents with the target type.  Supported: CVT_FP32_FP64, CVT_FP64_FP32,
// CVT_INT32_FP32, CVT_FP32_INT32 (round to nearest even, saturating), CVT_FP32_FP16, CVT_FP16_FP32; any other
// method, or a source of the wrong type, reports DECX_FAIL_INVALID_PARAM / DECX_FAIL_TYPE_MOT_MATCH.  Synchronous.
_DECX_API_ de::DH TypeCast(de::GPU_Matrix& src, de::GPU_Matrix& dst, const int cvt_method);
}  // namespace cuda
}  // namespace de
#endif
