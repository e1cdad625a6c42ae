// fp32 2-D convolution of a tensor with an array of kernels
// (reference: de::nn::cuda::Conv2D, srcs/modules/NN/convolution/CUDA/fp32/Conv2D.cu:34-131; the declaration in
// srcs/includes/DECX/nn/convolution.h is stale, the sample samples/Conv2D/Conv2D.cpp:98 calls this one).
//
//   dst(y, x, t) = sum_{i, j, c} src(y * strides.y + i - py, x * strides.x + j - px, c) * kernel_t(i, j, c)
// (a cross-correlation: no kernel flip).  _EXTEND_NONE_: py = px = 0, dst is (H - kh + 1) / sy rows of
// (W - kw + 1) / sx columns; _EXTEND_CONSTANT_: zero border of py = kh / 2, px = kw / 2, dst is H / sy rows of W / sx
// columns.  dst is re-shaped to (width, height, depth = number of kernels), fp32.  src and kernel must be fp32 with
// equal depth.  Synchronous; errors are returned and also recorded in de::GetLastError().
#ifndef DECX_B200_PUBLIC_NN_CONVOLUTION_H_
#define DECX_B200_PUBLIC_NN_CONVOLUTION_H_

#include "../basic.h"
#include "../basic_proc/VectorProc.h"
#include "../classes/GPU_Tensor.h"
#include "../classes/GPU_TensorArray.h"

namespace de {
namespace nn {
namespace cuda {
_DECX_API_ de::DH Conv2D(de::GPU_Tensor& src, de::GPU_TensorArray& kernel, de::GPU_Tensor& dst,
                         const de::Point2D strides = de::Point2D(1, 1),
                         const de::extend_label extend = de::extend_label::_EXTEND_NONE_);
}  // namespace cuda
}  // namespace nn
}  // namespace de
#endif
