// de::GPU_Matrix: abstract device matrix, row-major, rows `pitch` elements apart (width rounded up to
// 128 bytes).  Virtual order as in srcs/includes/DECX/classes/GPU_Matrix.h:19-47 (it differs from Matrix).
#ifndef DECX_B200_PUBLIC_GPU_MATRIX_H_
#define DECX_B200_PUBLIC_GPU_MATRIX_H_

#include "../basic.h"
#include "Matrix.h"

namespace de {

class _DECX_API_ GPU_Matrix {
public:
    GPU_Matrix() {}

    virtual uint Width() const = 0;
    virtual uint Height() const = 0;
    virtual void release() = 0;
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;
    virtual de::GPU_Matrix& SoftCopy(de::GPU_Matrix& src) = 0;
    virtual de::_DATA_FORMATS_ Format() const = 0;

    ~GPU_Matrix() {}
};

typedef const de::GPU_Matrix& InputGPUMatrix;
typedef de::GPU_Matrix& OutputGPUMatrix;
typedef de::GPU_Matrix& InOutGPUMatrix;

_DECX_API_ de::GPU_Matrix& CreateGPUMatrixRef();
_DECX_API_ de::GPU_Matrix* CreateGPUMatrixPtr();
_DECX_API_ de::GPU_Matrix* CreateGPUMatrixPtr(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width,
                                              const uint32_t _height, const de::_DATA_FORMATS_ format = de::_NA_);
_DECX_API_ de::GPU_Matrix& CreateGPUMatrixRef(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width,
                                              const uint32_t _height, const de::_DATA_FORMATS_ format = de::_NA_);

namespace cuda {
// page-lock / unlock the storage of a host matrix so that copies run at full PCIe speed
_DECX_API_ de::DH PinMemory(de::Matrix& src);
_DECX_API_ de::DH UnpinMemory(de::Matrix& src);
}
}  // namespace de
#endif
