// C-context exports of the drop-in (include/DECX/c_api.h): thin wrappers over the C++ API, same handle
// convention as the reference's own C exports (srcs/modules/core/classes/Matrix.cxx:279-305).
#include <cstring>

#include "../../include/DECX/c_api.h"
#include "internal.h"

static_assert(sizeof(DECX_Handle) == sizeof(de::DH), "the C and C++ error handles share one layout");
static_assert(sizeof(DECX_MatrixLayout) == sizeof(de::MatrixLayout), "the C and C++ layouts share one layout");

namespace {
decx::_Matrix* impl(DECX_Matrix m) { return reinterpret_cast<decx::_Matrix*>(m); }
int last() { return de::GetLastError()->error_type; }
}  // namespace

extern "C" {

DECX_Matrix DE_CreateEmptyMatrix(void) { return reinterpret_cast<DECX_Matrix>(new decx::_Matrix()); }

DECX_Matrix DE_CreateMatrix(const int8_t type, const uint32_t _width, const uint32_t _height, const int8_t format) {
    return reinterpret_cast<DECX_Matrix>(new decx::_Matrix(static_cast<de::_DATA_TYPES_FLAGS_>(type), _width, _height,
                                                            static_cast<de::_DATA_FORMATS_>(format)));
}

DECX_Handle DE_GetMatrixProp(const DECX_Matrix src, DECX_MatrixLayout* prop) {
    de::DH h;
    decx::err::success(&h);
    if (src == nullptr || prop == nullptr) decx::err::set(&h, de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
    else std::memcpy(prop, &impl(src)->_layout, sizeof(DECX_MatrixLayout));
    DECX_Handle out;
    std::memcpy(&out, &h, sizeof(out));
    return out;
}

int DE_InitCuda(void) {
    de::ResetLastError();
    de::InitCPUInfo();
    de::InitCuda();
    return last();
}
int DE_LastErrorType(void) { return last(); }
const char* DE_LastErrorString(void) { return de::GetLastError()->error_string; }

void* DE_GetMatrixData(DECX_Matrix m) { return m ? impl(m)->data : nullptr; }
int DE_PinMatrix(DECX_Matrix m) { return m ? de::cuda::PinMemory(*impl(m)).error_type : int(de::DECX_FAIL_INVALID_PARAM); }
int DE_UnpinMatrix(DECX_Matrix m) { return m ? de::cuda::UnpinMemory(*impl(m)).error_type : int(de::DECX_FAIL_INVALID_PARAM); }
void DE_ReleaseMatrix(DECX_Matrix m) {
    if (m == nullptr) return;
    delete impl(m);            // ~_Matrix releases the storage
}

int DE_GEMM_Host(DECX_Matrix A, DECX_Matrix B, DECX_Matrix C, DECX_Matrix dst) {
    if (A == nullptr || B == nullptr || dst == nullptr) return int(de::DECX_FAIL_INVALID_PARAM);
    de::ResetLastError();
    if (C != nullptr) de::blas::cuda::GEMM(*impl(A), *impl(B), *impl(C), *impl(dst));
    else de::blas::cuda::GEMM(*impl(A), *impl(B), *impl(dst));
    return last();
}

}  // extern "C"
