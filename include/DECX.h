// Umbrella header of the drop-in (the reference's srcs/includes/DECX.h pulls in every module; this one
// pulls in what the dense-GEMM path needs).
#ifndef DECX_B200_PUBLIC_DECX_H_
#define DECX_B200_PUBLIC_DECX_H_
#include "DECX/basic.h"
#include "DECX/classes/type_info.h"
#include "DECX/classes/class_utils.h"
#include "DECX/classes/DecxNumber.h"
#include "DECX/classes/Matrix.h"
#include "DECX/classes/GPU_Matrix.h"
#include "DECX/classes/Vector.h"
#include "DECX/classes/GPU_Vector.h"
#include "DECX/classes/Tensor.h"
#include "DECX/classes/TensorArray.h"
#include "DECX/classes/GPU_Tensor.h"
#include "DECX/classes/GPU_TensorArray.h"
#include "DECX/classes/decx_memcpy.h"
#include "DECX/BLAS/BLAS.h"
#include "DECX/basic_proc/type_cast.h"
#include "DECX/basic_proc/VectorProc.h"
#include "DECX/nn/convolution.h"
#endif
