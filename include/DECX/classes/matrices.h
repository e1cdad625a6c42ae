// Host and device matrix interfaces of the drop-in, in one place.
//
// Both are pure interfaces whose objects are made by the Create* factories and owned by the caller.  A program
// compiled against DECX's own headers calls the virtual functions by SLOT, so the order of the virtuals in each
// class is part of the binary contract and must not change:
//   de::Matrix      slots  Width, Height, release, SoftCopy, Type, Reinterpret, Format
//                   (srcs/includes/DECX/classes/Matrix.h:48-87)
//   de::GPU_Matrix  slots  Width, Height, release, Type, Reinterpret, SoftCopy, Format   <- not the same order
//                   (srcs/includes/DECX/classes/GPU_Matrix.h:19-47)
// de::Matrix additionally carries two "shadow" pointers right after the vptr; the header-inline element accessor
// ptr<T>(row, col) reads the implementation's data pointer and layout through them.
//
// Layout rules (rows are `pitch` elements apart):  host pitch = width rounded up to 32 bytes,
// device pitch = width rounded up to 128 bytes.  Constructors take (type, WIDTH, HEIGHT): width = columns.
#ifndef DECX_B200_PUBLIC_MATRICES_H_
#define DECX_B200_PUBLIC_MATRICES_H_

#include "../basic.h"
#include "class_utils.h"
#include "DecxNumber.h"

namespace de {

struct MatrixLayout {
    uint32_t width, height;
    uint32_t pitch;                 // elements per stored row
    int32_t _single_element_size;   // bytes
};
static_assert(sizeof(MatrixLayout) == 16, "de::MatrixLayout is part of the binary contract");

// ------------------------------------------------------------------------------------------ device matrix
class _DECX_API_ GPU_Matrix {
public:
    GPU_Matrix() {}

    virtual uint Width() const = 0;                                           // slot 0: columns
    virtual uint Height() const = 0;                                          // slot 1: rows
    virtual void release() = 0;                                               // slot 2: block back to the pool
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;                          // slot 3
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;     // slot 4: same bytes, other type
    virtual de::GPU_Matrix& SoftCopy(de::GPU_Matrix& src) = 0;                // slot 5: share src's storage
    virtual de::_DATA_FORMATS_ Format() const = 0;                            // slot 6

    ~GPU_Matrix() {}
};

// ------------------------------------------------------------------------------------------ host matrix
class _DECX_API_ Matrix {
protected:
    _SHADOW_ATTRIBUTE_(void*) _exp_data_ptr;                 // -> the implementation's data pointer
    _SHADOW_ATTRIBUTE_(de::MatrixLayout) _exp_matrix_dscr;   // -> the implementation's layout

public:
    Matrix() {}

    virtual uint32_t Width() const = 0;                                       // slot 0: columns
    virtual uint32_t Height() const = 0;                                      // slot 1: rows

    // address of element (row, col); _ptr_type must be the element type
    template <typename _ptr_type>
    _ptr_type* ptr(const int row, const int col) {
        return static_cast<_ptr_type*>(*this->_exp_data_ptr) + size_t(this->_exp_matrix_dscr->pitch) * row + col;
    }

    virtual void release() = 0;                                               // slot 2
    virtual de::Matrix& SoftCopy(de::Matrix& src) = 0;                        // slot 3
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;                          // slot 4
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;     // slot 5
    virtual de::_DATA_FORMATS_ Format() const = 0;                            // slot 6

    ~Matrix() {}
};

typedef const de::Matrix& InputMatrix;
typedef de::Matrix& OutputMatrix;
typedef de::Matrix& InOutMatrix;
typedef const de::GPU_Matrix& InputGPUMatrix;
typedef de::GPU_Matrix& OutputGPUMatrix;
typedef de::GPU_Matrix& InOutGPUMatrix;

// ------------------------------------------------------------------------------------------ factories
// Empty objects (shaped later, e.g. by GEMM for its result) and shaped, zero-filled ones.
_DECX_API_ de::Matrix* CreateMatrixPtr();
_DECX_API_ de::Matrix& CreateMatrixRef();
_DECX_API_ de::GPU_Matrix* CreateGPUMatrixPtr();
_DECX_API_ de::GPU_Matrix& CreateGPUMatrixRef();
_DECX_API_ de::Matrix* CreateMatrixPtr(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width, const uint32_t _height,
                                       const de::_DATA_FORMATS_ format = de::_NA_);
_DECX_API_ de::Matrix& CreateMatrixRef(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width, const uint32_t _height,
                                       const de::_DATA_FORMATS_ format = de::_NA_);
_DECX_API_ de::GPU_Matrix* CreateGPUMatrixPtr(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width,
                                              const uint32_t _height, const de::_DATA_FORMATS_ format = de::_NA_);
_DECX_API_ de::GPU_Matrix& CreateGPUMatrixRef(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width,
                                              const uint32_t _height, const de::_DATA_FORMATS_ format = de::_NA_);

namespace cuda {
// page-lock / unlock the storage of a host matrix so that copies run at full PCIe speed
_DECX_API_ de::DH PinMemory(de::Matrix& src);
_DECX_API_ de::DH UnpinMemory(de::Matrix& src);
}  // namespace cuda
}  // namespace de
#endif
