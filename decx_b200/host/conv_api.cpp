// de::nn::cuda::Conv2D on device tensors.
//
// Reference flow (srcs/modules/NN/convolution/CUDA/fp32/Conv2D.cu:57-131): pooled stream + event, a cached planner
// that owns the im2col, extended-source and transposed-kernel buffers, dst re-shaped to (OW, OH, number of kernels),
// im2col + its own fp32 GEMM kernel per fragment of rows, event wait.  The flow and error codes are kept; the work is
// decxb200_conv2d_fp32 (include/decx_b200.h: implicit GEMM on the tensor cores) with one scratch block from the
// device pool per call, and nothing calls exit().
#include <cstring>

#include "../../include/decx_b200.h"
#include "internal.h"

namespace {
de::DH fail(int code, const char* msg) {
    de::DH h;
    decx::err::set(&h, code, msg);
    decx::err::set(de::GetLastError(), code, msg);
    return h;
}
}  // namespace

de::DH de::nn::cuda::Conv2D(de::GPU_Tensor& src, de::GPU_TensorArray& kernel, de::GPU_Tensor& dst, const de::Point2D strides,
                            const de::extend_label extend) {
    de::DH handle;
    decx::err::success(&handle);
    if (!decx::cuda::_is_CUDA_init()) return fail(de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first");
    decx::_GPU_Tensor* s = dynamic_cast<decx::_GPU_Tensor*>(&src);
    decx::_GPU_TensorArray* k = dynamic_cast<decx::_GPU_TensorArray*>(&kernel);
    decx::_GPU_Tensor* d = dynamic_cast<decx::_GPU_Tensor*>(&dst);
    if (s == nullptr || k == nullptr || d == nullptr || !s->_init || !k->_init)
        return fail(de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    if (s->Type() != de::_FP32_ || k->Type() != de::_FP32_)
        return fail(de::DECX_FAIL_UNSUPPORTED_TYPE, "error: The data type is not supported by the convolution");
    if (s->Depth() != k->Depth()) return fail(de::DECX_FAIL_DimsNotMatching, "error: Dim(s) is(are) not equal to each other");
    if (d == s) return fail(de::DECX_FAIL_INVALID_PARAM, "error: dst must not be the source");
    if (extend != de::_EXTEND_NONE_ && extend != de::_EXTEND_CONSTANT_)
        return fail(de::DECX_FAIL_ErrorFlag, "error: This flag is meaningless in current context");
    if (strides.x <= 0 || strides.y <= 0) return fail(de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
    if (s->_device != k->_device) return fail(de::DECX_FAIL_INVALID_PARAM, "error: The operands live on different devices");

    const uint32_t H = s->Height(), W = s->Width(), C = s->Depth(), kh = k->Height(), kw = k->Width(), n = k->TensorNum();
    const uint32_t sx = uint32_t(strides.x), sy = uint32_t(strides.y);
    const int ext = (extend == de::_EXTEND_NONE_) ? DECXB200_EXTEND_NONE : DECXB200_EXTEND_CONSTANT;
    uint32_t OH = 0, OW = 0;
    if (decxb200_conv2d_fp32_out_dims(H, W, kh, kw, sx, sy, ext, &OH, &OW) != 0)
        return fail(de::DECX_FAIL_DimsNotMatching, "error: The kernel does not fit the source");

    int cur = 0;
    cudaGetDevice(&cur);
    if (cur != s->_device) cudaSetDevice(s->_device);
    struct Restore {
        int to, from;
        ~Restore() { if (to != from) cudaSetDevice(to); }
    } restore{cur, s->_device};

    decx::cuda_stream* S = decx::cuda::get_cuda_stream_ptr(cudaStreamNonBlocking);
    if (S == nullptr) return fail(de::DECX_FAIL_CUDA_STREAM, "error: Fail to access cuda stream");
    decx::cuda_event* E = decx::cuda::get_cuda_event_ptr(cudaEventBlockingSync);
    if (E == nullptr) {
        S->detach();
        return fail(de::DECX_FAIL_CUDA_EVENT, "error: Fail to access cuda event");
    }
    d->re_construct(de::_FP32_, OW, OH, n, S);
    decx::PtrInfo<void> ws;
    int rc = 0;
    const char* what = nullptr;
    if (!d->_init) {
        rc = de::DECX_FAIL_CUDA_ALLOCATION;
        what = "error: Fail to allocate memory on device";
    } else {
        const size_t need = decxb200_conv2d_fp32_workspace_bytes(H, W, C, kh, kw, n, sx, sy, ext, d->_layout.wpitch,
                                                                 d->_layout.dpitch);
        if (decx::alloc::_device_malloc(&ws, need, false, S) != 0) {
            cudaGetLastError();
            rc = de::DECX_FAIL_CUDA_ALLOCATION;
            what = "error: Fail to allocate memory on device";
        } else {
            const int c = decxb200_conv2d_fp32(S->get_raw_stream_ref(), s->Tens.ptr, H, W, C, s->_layout.wpitch, s->_layout.dpitch,
                                               k->TensArr.ptr, kh, kw, n, k->_layout.wpitch, k->_layout.dpitch, k->_gap,
                                               d->Tens.ptr, d->_layout.wpitch, d->_layout.dpitch, sx, sy, ext, ws.ptr, need,
                                               nullptr);
            if (c != 0) {
                rc = c < 0 ? de::DECX_FAIL_INVALID_PARAM : de::DECX_FAIL_CUDA_STREAM;
                what = decxb200_strerror(c);
            }
        }
    }
    E->event_record(S);
    E->synchronize();
    decx::alloc::_device_dealloc(&ws);
    E->detach();
    S->detach();
    if (rc != 0) return fail(rc, what);
    return handle;
}
