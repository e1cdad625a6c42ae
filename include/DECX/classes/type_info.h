// Element-type and format flags; values as in the reference's srcs/includes/DECX/classes/type_info.h:20-54.
#ifndef DECX_B200_PUBLIC_TYPE_INFO_H_
#define DECX_B200_PUBLIC_TYPE_INFO_H_

namespace de {
enum _DATA_TYPES_FLAGS_ {
    _VOID_ = 0,
    _FP32_ = 1,
    _FP64_ = 2,
    _FP16_ = 3,
    _INT32_ = 4,
    _COMPLEX_F32_ = 5,
    _COMPLEX_F64_ = 6,
    _UINT64_ = 7,
    _UINT8_ = 8,
    _UCHAR4_ = 12,
    _VECTOR3F_ = 14,
    _VECTOR4F_ = 15
};

enum _DATA_FORMATS_ { _NA_ = 0, _RGB_ = 1, _YUV444_ = 2, _HSV_ = 3, _CPLX_CARTESIAN_ = 4, _CPLX_POLAR_ = 5 };
}  // namespace de
#endif
