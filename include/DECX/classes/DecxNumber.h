// de::Number: a tagged scalar passed BY VALUE to the fused GEMM (alpha, beta).  32 bytes: a 16-byte
// aligned union followed by the type flag, as in srcs/includes/DECX/classes/DecxNumber.h:27-186.
#ifndef DECX_B200_PUBLIC_NUMBER_H_
#define DECX_B200_PUBLIC_NUMBER_H_

#include "class_utils.h"

namespace de {
_DECX_API_ de::Half Float2Half(const float& __x);
_DECX_API_ float Half2Float(const de::Half& __x);

class _DECX_API_ Number {
private:
    union __align__(16) _data {
        float _fp32;
        double _fp64;
        de::CPf _cplxf32;
        de::CPd _cplxd64;
        uint8_t _u8;
        int32_t _i32;
        de::Half _fp16;
        _data() : _cplxd64(0.0, 0.0) {}
    };
    _data _number;
    int32_t _data_type_flag;

public:
    Number() : _data_type_flag(de::_VOID_) {}
    Number(const int32_t v) : _data_type_flag(de::_INT32_) { _number._i32 = v; }
    Number(const uint8_t v) : _data_type_flag(de::_UINT8_) { _number._u8 = v; }
    Number(const float v) : _data_type_flag(de::_FP32_) { _number._fp32 = v; }
    Number(const double v) : _data_type_flag(de::_FP64_) { _number._fp64 = v; }
    Number(const de::Half v) : _data_type_flag(de::_FP16_) { _number._fp16 = v; }
    Number(const de::CPf v) : _data_type_flag(de::_COMPLEX_F32_) { _number._cplxf32 = v; }
    Number(const de::CPd v) : _data_type_flag(de::_COMPLEX_F64_) { _number._cplxd64 = v; }

    int32_t Type() const { return _data_type_flag; }

    template <typename _Ty>
    _Ty get_data() { return *reinterpret_cast<_Ty*>(&this->_number); }
    template <typename _Ty>
    const _Ty& get_data_ref() const { return *reinterpret_cast<const _Ty*>(&this->_number); }

    de::Number& operator=(const float v) { _number._fp32 = v; _data_type_flag = de::_FP32_; return *this; }
    de::Number& operator=(const double v) { _number._fp64 = v; _data_type_flag = de::_FP64_; return *this; }
    de::Number& operator=(const de::CPf v) { _number._cplxf32 = v; _data_type_flag = de::_COMPLEX_F32_; return *this; }
    de::Number& operator=(const de::CPd v) { _number._cplxd64 = v; _data_type_flag = de::_COMPLEX_F64_; return *this; }
    de::Number& operator=(const uint8_t v) { _number._u8 = v; _data_type_flag = de::_UINT8_; return *this; }
    de::Number& operator=(const int32_t v) { _number._i32 = v; _data_type_flag = de::_INT32_; return *this; }
    de::Number& operator=(const de::Half v) { _number._fp16 = v; _data_type_flag = de::_FP16_; return *this; }
};

typedef const de::Number& InputNumber;
typedef de::Number& OutputNumber;
}  // namespace de
#endif
