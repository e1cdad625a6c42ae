/*
 * C-context view of the drop-in: what a C program, or a binding from another language, calls.
 *
 * DE_CreateEmptyMatrix / DE_CreateMatrix / DE_GetMatrixProp are the reference's own C exports
 * (srcs/includes/DECX/classes/Matrix.h:118-141, srcs/modules/core/classes/Matrix.cxx:279-305).  The reference stops
 * there: its C context can make a matrix but cannot fill, pin, multiply or release one.  The rest of this header
 * closes that gap for the GEMM path with the same handle convention (an opaque pointer to the implementation
 * object).  Every function that can fail returns the error code that de::GetLastError() would hold (0 = success);
 * DE_LastErrorString() gives the message.
 */
#ifndef DECX_B200_PUBLIC_C_API_H_
#define DECX_B200_PUBLIC_C_API_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DECX_C_API __attribute__((visibility("default")))
#else
#define DECX_C_API
#endif

typedef struct DECX_MatrixLayout_t {
    uint32_t _width, _height;
    uint32_t _pitch;
    int32_t _single_element_size;
} DECX_MatrixLayout;

typedef struct DECX_Handle_t {
    int error_type;
    char error_string[100];
} DECX_Handle;

typedef struct DECX_Matrix_t* DECX_Matrix;

/* the reference's C exports */
DECX_C_API DECX_Matrix DE_CreateEmptyMatrix(void);
DECX_C_API DECX_Matrix DE_CreateMatrix(const int8_t type, const uint32_t _width, const uint32_t _height, const int8_t format);
DECX_C_API DECX_Handle DE_GetMatrixProp(const DECX_Matrix src, DECX_MatrixLayout* prop);

/* start-up (de::InitCuda + de::InitCPUInfo) and the error handle */
DECX_C_API int DE_InitCuda(void);
DECX_C_API int DE_LastErrorType(void);
DECX_C_API const char* DE_LastErrorString(void);

/* storage of a host matrix: first element of row 0; rows are _pitch elements apart */
DECX_C_API void* DE_GetMatrixData(DECX_Matrix m);
DECX_C_API int DE_PinMatrix(DECX_Matrix m);       /* de::cuda::PinMemory   */
DECX_C_API int DE_UnpinMatrix(DECX_Matrix m);     /* de::cuda::UnpinMemory */
DECX_C_API void DE_ReleaseMatrix(DECX_Matrix m);  /* release() and delete the object */

/* de::blas::cuda::GEMM on host matrices: dst = A . B, or dst = A . B + C when C is not NULL */
DECX_C_API int DE_GEMM_Host(DECX_Matrix A, DECX_Matrix B, DECX_Matrix C, DECX_Matrix dst);

#ifdef __cplusplus
}
#endif
#endif
