// Border modes shared by the extension and convolution APIs
// (reference: srcs/includes/DECX/basic_proc/VectorProc.h:22-26).  Only the enumeration is part of this library.
#ifndef DECX_B200_PUBLIC_VECTORPROC_H_
#define DECX_B200_PUBLIC_VECTORPROC_H_

namespace de {
enum extend_label {
    _EXTEND_NONE_ = 0,
    _EXTEND_REFLECT_ = 1,
    _EXTEND_CONSTANT_ = 2,
};
}  // namespace de
#endif
