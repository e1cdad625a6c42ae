// Host and device vector interfaces of the drop-in (operands of the Vector overloads of de::blas::cuda::GEMM).
//
// Pure interfaces made by the Create* factories and owned by the caller; virtual slot order is part of the
// binary contract:
//   de::Vector      slots  Len, release, SoftCopy, Type, Reinterpret; one shadow pointer after the vptr for the
//                   header-inline ptr<T>(i)            (srcs/includes/DECX/classes/Vector.h:20-56)
//   de::GPU_Vector  slots  Len, release, SoftCopy, Type, Reinterpret      (srcs/includes/DECX/classes/GPU_Vector.h:19-43)
// Storage is padded to a whole number of 16-byte groups (host: 8 elements, device: 4, as in the reference's
// `_length`), zero-filled.
#ifndef DECX_B200_PUBLIC_VECTORS_H_
#define DECX_B200_PUBLIC_VECTORS_H_

#include "../basic.h"
#include "class_utils.h"

namespace de {

class _DECX_API_ Vector {
protected:
    _SHADOW_ATTRIBUTE_(void*) _exp_data_ptr;                 // -> the implementation's data pointer

public:
    Vector() {}

    virtual size_t Len() const = 0;                                           // slot 0

    template <typename _ptr_type>
    _ptr_type* ptr(const uint64_t _idx) {
        return static_cast<_ptr_type*>(*this->_exp_data_ptr) + _idx;
    }

    virtual void release() = 0;                                               // slot 1
    virtual de::Vector& SoftCopy(de::Vector& src) = 0;                        // slot 2
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;                          // slot 3
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;     // slot 4

    ~Vector() {}
};

class _DECX_API_ GPU_Vector {
public:
    GPU_Vector() {}

    virtual size_t Len() const = 0;                                           // slot 0
    virtual void release() = 0;                                               // slot 1
    virtual de::GPU_Vector& SoftCopy(de::GPU_Vector& src) = 0;                // slot 2
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;                          // slot 3
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;     // slot 4

    ~GPU_Vector() {}
};

typedef const de::Vector& InputVector;
typedef de::Vector& OutputVector;
typedef de::Vector& InOutVector;

_DECX_API_ de::Vector& CreateVectorRef();
_DECX_API_ de::Vector* CreateVectorPtr();
_DECX_API_ de::Vector& CreateVectorRef(const de::_DATA_TYPES_FLAGS_ _type, size_t len);
_DECX_API_ de::Vector* CreateVectorPtr(const de::_DATA_TYPES_FLAGS_ _type, size_t len);
_DECX_API_ de::GPU_Vector& CreateGPUVectorRef();
_DECX_API_ de::GPU_Vector* CreateGPUVectorPtr();
_DECX_API_ de::GPU_Vector& CreateGPUVectorRef(const de::_DATA_TYPES_FLAGS_ _type, const size_t _length);
_DECX_API_ de::GPU_Vector* CreateGPUVectorPtr(const de::_DATA_TYPES_FLAGS_ _type, const size_t _length);

namespace cuda {
_DECX_API_ de::DH PinMemory(de::Vector& src);
_DECX_API_ de::DH UnpinMemory(de::Vector& src);
}  // namespace cuda
}  // namespace de
#endif
