// Source compatibility: DECX programs include "DECX/classes/Matrix.h".  The declarations live in matrices.h.
#ifndef DECX_B200_PUBLIC_MATRIX_H_
#define DECX_B200_PUBLIC_MATRIX_H_
#include "matrices.h"
#endif
