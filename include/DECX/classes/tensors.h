// Host and device tensor interfaces of the drop-in (operands of de::nn::cuda::Conv2D).
//
// A tensor is stored channels-innermost: element (row, column, channel) at
//     base[row * dp_x_wp + column * dpitch + channel]
// with dpitch = depth rounded up to 16 bytes' worth of elements and wpitch = width rounded up to 4 (host) or 8
// (device) columns, dp_x_wp = dpitch * wpitch, zero-filled
// (srcs/common/Classes/Tensor.h:59-82, srcs/modules/core/classes/Tensor.cxx:40-70, GPU_Tensor.cu:35-88).
// A tensor array is `tensor_num` such tensors of one shape, back to back.
//
// Pure interfaces made by the Create* factories and owned by the caller; virtual slot order and the shadow members
// behind the header-inline ptr<T>() are part of the binary contract:
//   de::Tensor           Width, Height, Depth, SoftCopy, release, Type, Reinterpret
//                        (srcs/includes/DECX/classes/Tensor.h:54-104)
//   de::TensorArray      Width, Height, Depth, TensorNum, SoftCopy, Type, Reinterpret, Extract_SoftCopy, release
//                        (srcs/includes/DECX/classes/TensorArray.h:19-67)
//   de::GPU_Tensor       Width, Height, Depth, SoftCopy, release, Type, Reinterpret, Extract_SoftCopy
//                        (srcs/includes/DECX/classes/GPU_Tensor.h:19-47)
//   de::GPU_TensorArray  Width, Height, Depth, TensorNum, Type, Reinterpret, SoftCopy, Extract_SoftCopy, release
//                        (srcs/includes/DECX/classes/GPU_TensorArray.h:22-52)
#ifndef DECX_B200_PUBLIC_TENSORS_H_
#define DECX_B200_PUBLIC_TENSORS_H_

#include "../basic.h"
#include "class_utils.h"
#include "matrices.h"

namespace de {

struct TensorLayout {
    uint32_t width, height, depth;
    uint32_t dpitch;                // elements between neighbouring columns
    uint32_t wpitch;                // columns per stored row
    uint64_t dp_x_wp;               // elements between neighbouring rows
    uint8_t _single_element_size;
    uint64_t plane[3];              // active elements of the WH, WD and HD planes
};

class _DECX_API_ Tensor {
protected:
    _SHADOW_ATTRIBUTE_(void*) _exp_data_ptr;
    _SHADOW_ATTRIBUTE_(de::TensorLayout) _exp_tensor_dscr;

public:
    Tensor() {}

    virtual uint32_t Width() const = 0;                                       // slot 0
    virtual uint32_t Height() const = 0;                                      // slot 1
    virtual uint32_t Depth() const = 0;                                       // slot 2

    // (row, column, channel)
    template <typename _ptr_type>
    _ptr_type* ptr(const int x, const int y, const int z) {
        return static_cast<_ptr_type*>(*this->_exp_data_ptr) +
               (uint64_t(x) * this->_exp_tensor_dscr->dp_x_wp + uint64_t(y) * this->_exp_tensor_dscr->dpitch + z);
    }

    virtual de::Tensor& SoftCopy(de::Tensor& src) = 0;                        // slot 3
    virtual void release() = 0;                                               // slot 4
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;                          // slot 5
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;     // slot 6
};

class _DECX_API_ TensorArray {
protected:
    _SHADOW_ATTRIBUTE_(void**) _exp_data_ptr;                // -> the array of the tensors' base pointers
    _SHADOW_ATTRIBUTE_(de::TensorLayout) _exp_tensor_dscr;

public:
    TensorArray() {}

    virtual uint32_t Width() const = 0;                                       // slot 0
    virtual uint32_t Height() const = 0;                                      // slot 1
    virtual uint32_t Depth() const = 0;                                       // slot 2
    virtual uint32_t TensorNum() const = 0;                                   // slot 3

    // (row, column, channel, tensor)
    template <typename _ptr_type>
    _ptr_type* ptr(const int x, const int y, const int z, const int tensor_id) {
        return static_cast<_ptr_type*>((*this->_exp_data_ptr)[tensor_id]) + uint64_t(x) * this->_exp_tensor_dscr->dp_x_wp +
               uint64_t(y) * this->_exp_tensor_dscr->dpitch + z;
    }

    virtual de::TensorArray& SoftCopy(de::TensorArray& src) = 0;              // slot 4
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;                          // slot 5
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;     // slot 6
    virtual de::DH Extract_SoftCopy(const uint32_t index, de::Tensor& dst) const = 0;   // slot 7
    virtual void release() = 0;                                               // slot 8
};

class _DECX_API_ GPU_Tensor {
public:
    GPU_Tensor() {}

    virtual uint32_t Width() const = 0;                                       // slot 0
    virtual uint32_t Height() const = 0;                                      // slot 1
    virtual uint32_t Depth() const = 0;                                       // slot 2
    virtual de::GPU_Tensor& SoftCopy(de::GPU_Tensor& src) = 0;                // slot 3
    virtual void release() = 0;                                               // slot 4
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;                          // slot 5
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;     // slot 6
    virtual de::DH Extract_SoftCopy(const uint32_t index, de::GPU_Tensor& dst) const = 0;   // slot 7
};

class _DECX_API_ GPU_TensorArray {
public:
    GPU_TensorArray() {}

    virtual uint32_t Width() const = 0;                                       // slot 0
    virtual uint32_t Height() const = 0;                                      // slot 1
    virtual uint32_t Depth() const = 0;                                       // slot 2
    virtual uint32_t TensorNum() const = 0;                                   // slot 3
    virtual de::_DATA_TYPES_FLAGS_ Type() const = 0;                          // slot 4
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) = 0;     // slot 5
    virtual de::GPU_TensorArray& SoftCopy(const de::GPU_TensorArray& src) = 0;   // slot 6
    virtual de::DH Extract_SoftCopy(const uint32_t index, de::GPU_Tensor& dst) const = 0;   // slot 7
    virtual void release() = 0;                                               // slot 8
};

_DECX_API_ de::Tensor* CreateTensorPtr();
_DECX_API_ de::Tensor& CreateTensorRef();
_DECX_API_ de::Tensor* CreateTensorPtr(const de::_DATA_TYPES_FLAGS_ _type, const uint32_t _width, const uint32_t _height,
                                       const uint32_t _depth);
_DECX_API_ de::Tensor& CreateTensorRef(const de::_DATA_TYPES_FLAGS_ _type, const uint32_t _width, const uint32_t _height,
                                       const uint32_t _depth);
_DECX_API_ de::TensorArray& CreateTensorArrayRef();
_DECX_API_ de::TensorArray* CreateTensorArrayPtr();
_DECX_API_ de::TensorArray& CreateTensorArrayRef(const de::_DATA_TYPES_FLAGS_ _type, const uint32_t width, const uint32_t height,
                                                 const uint32_t depth, const uint32_t tensor_num);
_DECX_API_ de::TensorArray* CreateTensorArrayPtr(const de::_DATA_TYPES_FLAGS_ _type, const uint32_t width, const uint32_t height,
                                                 const uint32_t depth, const uint32_t tensor_num);
_DECX_API_ de::GPU_Tensor* CreateGPUTensorPtr();
_DECX_API_ de::GPU_Tensor& CreateGPUTensorRef();
_DECX_API_ de::GPU_Tensor* CreateGPUTensorPtr(const de::_DATA_TYPES_FLAGS_ _type, const uint32_t _width, const uint32_t _height,
                                              const uint32_t _depth);
_DECX_API_ de::GPU_Tensor& CreateGPUTensorRef(const de::_DATA_TYPES_FLAGS_ _type, const uint32_t _width, const uint32_t _height,
                                              const uint32_t _depth);
_DECX_API_ de::GPU_TensorArray& CreateGPUTensorArrayRef();
_DECX_API_ de::GPU_TensorArray* CreateGPUTensorArrayPtr();
_DECX_API_ de::GPU_TensorArray& CreateGPUTensorArrayRef(const de::_DATA_TYPES_FLAGS_ _type, const uint32_t width,
                                                        const uint32_t height, const uint32_t depth,
                                                        const uint32_t _array_length);
_DECX_API_ de::GPU_TensorArray* CreateGPUTensorArrayPtr(const de::_DATA_TYPES_FLAGS_ _type, const uint32_t width,
                                                        const uint32_t height, const uint32_t depth,
                                                        const uint32_t _array_length);

namespace cuda {
_DECX_API_ de::DH PinMemory(de::Tensor& src);
_DECX_API_ de::DH UnpinMemory(de::Tensor& src);
}  // namespace cuda
}  // namespace de
#endif
