// Include-path compatibility: the vector interfaces live in vectors.h.
#ifndef DECX_B200_PUBLIC_VECTOR_H_
#define DECX_B200_PUBLIC_VECTOR_H_
#include "vectors.h"
#endif
