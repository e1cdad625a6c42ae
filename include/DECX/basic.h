// Public basics of the drop-in: export macro, the error handle de::DH, library start-up calls.
// Layout- and name-compatible with the reference's srcs/includes/DECX/basic.h for everything the GEMM
// path touches; the error codes are the ones the reference library really writes
// (srcs/common/Handle/decx_handle.h:47-179), not the stale public copy.
#ifndef DECX_B200_PUBLIC_BASIC_H_
#define DECX_B200_PUBLIC_BASIC_H_

#include <cstddef>
#include <cstdint>
#include <cstdio>

typedef unsigned char uchar;
typedef unsigned int uint;

#define _DECX_API_ __attribute__((visibility("default")))
#ifndef __align__
#define __align__(n) __attribute__((aligned(n)))
#endif
// members of the public base classes that mirror private state of the implementation objects
#define _SHADOW_ATTRIBUTE_(__actual_type) __actual_type*

namespace de {

// 104 bytes: code + message.  One process-wide instance is read with de::GetLastError().
typedef struct DECX_Handle {
    int error_type;
    char error_string[100];
} DH;

enum DECX_error_types {
    DECX_SUCCESS = 0x00,
    DECX_FAIL_CPU_not_init = 0x01,
    DECX_FAIL_FFT_error_length = 0x02,
    DECX_FAIL_DimsNotMatching = 0x03,
    DECX_FAIL_Complex_comparing = 0x04,
    DECX_FAIL_ConvBadKernel = 0x05,
    DECX_FAIL_CVNLM_BadArea = 0x06,
    DECX_FAIL_ErrorFlag = 0x07,
    DECX_FAIL_ALLOCATION = 0x08,
    DECX_FAIL_CUDA_STREAM = 0x09,
    DECX_FAIL_CLASS_NOT_INIT = 0x0a,
    DECX_FAIL_TYPE_MOT_MATCH = 0x0b,
    DECX_FAIL_INVALID_PARAM = 0x0c,
    DECX_FAIL_IMAGE_LOAD_FAILED = 0x0d,
    DECX_FAIL_CUDA_EVENT = 0x0e,
    MULTIPLE_REFERENCES = 0x0f,
    CPU_HYPER_THREADING = 0x10,
    MEMCPY_DIFFERENT_TYPES = 0x11,
    DECX_FAIL_MEMCPY_OVERRANGED = 0x12,
    DECX_FAIL_UNSUPPORTED_TYPE = 0x13,
    DECX_FAIL_HOST_MEM_REGISTERED = 0x14,
    DECX_FAIL_HOST_MEM_UNREGISTERED = 0x15,
    DECX_FAIL_CUDA_not_init = 0x16,
    DECX_FAIL_CUDA_ALLOCATION = 0x17
};

// Caches the properties of the CURRENT device; call before anything that touches the GPU
// (reference: srcs/modules/core/configs/config.cu:35-40).
_DECX_API_ void InitCuda();
// Records the host's logical CPU count (reference: config.cxx:35-41; no CPUID assembly here).
_DECX_API_ void InitCPUInfo();

namespace cuda {
// Returns every pooled device block, stream and event to CUDA.
_DECX_API_ void DECX_CUDA_exit();
}
namespace cpu {
_DECX_API_ void DecxSetThreadingNum(const uint64_t _thread_num);
}

// The process-wide error handle.  GEMM entry points return void and report here; like the reference's
// CUDA GEMM they do not reset it on success (srcs/modules/BLAS/GEMM/CUDA/GEMM_LS.cu:315-393).
_DECX_API_ de::DH* GetLastError();
_DECX_API_ void ResetLastError();

}  // namespace de
#endif
