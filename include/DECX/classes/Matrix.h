// de::Matrix: abstract host matrix, row-major, rows `pitch` elements apart (width rounded up to 32 bytes).
// Same member order and virtual-function order as srcs/includes/DECX/classes/Matrix.h:48-87, so code
// compiled against either header calls the same slots.
#ifndef DECX_B200_PUBLIC_MATRIX_H_
#define DECX_B200_PUBLIC_MATRIX_H_

#include "../basic.h"
#include "class_utils.h"
#include "DecxNumber.h"

namespace de {

struct MatrixLayout {
    uint32_t width, height;
    uint32_t pitch;                 // elements per stored row
    int32_t _single_element_size;   // bytes
};

class _DECX_API_ Matrix {
protected:
    _SHADOW_ATTRIBUTE_(void*) _exp_data_ptr;                 // -> the implementation's data pointer
    _SHADOW_ATTRIBUTE_(de::MatrixLayout) _exp_matrix_dscr;   // -> the implementation's layout

public:
    Matrix() {}

    virtual uint32_t Width() const = 0;    // columns
    virtual uint32_t Height() const = 0;   // rows

    // element (row, col); _ptr_type must be the element type
    template <typename _ptr_type>
    _ptr_type* ptr(const int row, const int col) {
        return static_cast<_ptr_type*>(*this->_exp_data_ptr) + size_t(this->_exp_matrix_dscr->pitch) * row + col;
    }

    virtual void release() = 0;
    virtual de::Matrix& SoftCopy(de::Matrix& src) = 0;
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;
    virtual de::_DATA_FORMATS_ Format() const = 0;

    ~Matrix() {}
};

typedef const de::Matrix& InputMatrix;
typedef de::Matrix& OutputMatrix;
typedef de::Matrix& InOutMatrix;

// Constructors take (type, WIDTH, HEIGHT): width = number of columns.  The caller owns the object.
_DECX_API_ de::Matrix* CreateMatrixPtr();
_DECX_API_ de::Matrix& CreateMatrixRef();
_DECX_API_ de::Matrix* CreateMatrixPtr(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width, const uint32_t _height,
                                       const de::_DATA_FORMATS_ format = de::_NA_);
_DECX_API_ de::Matrix& CreateMatrixRef(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width, const uint32_t _height,
                                       const de::_DATA_FORMATS_ format = de::_NA_);
}  // namespace de
#endif
