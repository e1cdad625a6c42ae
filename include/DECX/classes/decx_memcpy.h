// de::Memcpy between a host and a device matrix (reference: srcs/includes/DECX/classes/decx_memcpy.h:42-53).
#ifndef DECX_B200_PUBLIC_MEMCPY_H_
#define DECX_B200_PUBLIC_MEMCPY_H_

#include "Matrix.h"
#include "GPU_Matrix.h"
#include "Vector.h"
#include "GPU_Vector.h"
#include "Tensor.h"
#include "GPU_Tensor.h"

namespace de {
enum DECX_Memcpy_Flags { DECX_MEMCPY_H2D = 0, DECX_MEMCPY_D2H = 1 };

// The host object is always the first argument.  Points are {x = column, y = row}; cpy_size = {W, H}.
// start_src / start_dst are the corners in the SOURCE / DESTINATION of the chosen direction.  Synchronous.
_DECX_API_ de::DH Memcpy(de::Matrix& __host, de::GPU_Matrix& __device, const de::Point2D start_src,
                         de::Point2D start_dst, const de::Point2D cpy_size, const int _memcpy_flag);
// Vectors: cpy_size elements from index start_src of the source to index start_dst of the destination.
_DECX_API_ de::DH Memcpy(de::Vector& __host, de::GPU_Vector& __device, const uint64_t start_src, const uint64_t start_dst,
                         const uint64_t cpy_size, const int _memcpy_flag);
// Tensors: points are {x = channel, y = column, z = row}; cpy_size = {D, W, H}.
_DECX_API_ de::DH Memcpy(de::Tensor& __host, de::GPU_Tensor& __device, const de::Point3D start_src,
                         const de::Point3D start_dst, const de::Point3D cpy_size, const int _memcpy_flag);
}  // namespace de
#endif
