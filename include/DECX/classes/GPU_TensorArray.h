// Include-path compatibility: the tensor interfaces live in tensors.h.
#ifndef DECX_B200_PUBLIC_GPU_TENSORARRAY_H_
#define DECX_B200_PUBLIC_GPU_TENSORARRAY_H_
#include "tensors.h"
#endif
