// Matrix-vector overloads of de::blas::cuda::GEMM, de::cuda::Transpose and de::cuda::TypeCast.
//
// Reference flows: VMM (srcs/modules/BLAS/GEMM/CUDA/VMM.cu:55-184: pooled stream + event, device staging of the
// host matrix and vector, kernel(s), copy of the result, event wait), Transpose
// (srcs/modules/BLAS/Basic_process/transpose/transpose.cu:50-101) and TypeCast
// (srcs/modules/BLAS/Basic_process/type_cast/GPU_Matrix_type_cast.cu:38-85).  The flows and error codes are kept;
// the kernels are the ones behind include/decx_b200.h, and nothing calls exit().
#include <cstring>

#include "../../include/decx_b200.h"
#include "internal.h"

namespace {

void fail(int code, const char* msg) { decx::err::set(de::GetLastError(), code, msg); }

struct StreamEvent {      // pooled stream + blocking-sync event for one synchronous call
    decx::cuda_stream* S = nullptr;
    decx::cuda_event* E = nullptr;
    bool ok() {
        S = decx::cuda::get_cuda_stream_ptr(cudaStreamNonBlocking);
        if (S == nullptr) { fail(de::DECX_FAIL_CUDA_STREAM, "error: Fail to access cuda stream"); return false; }
        E = decx::cuda::get_cuda_event_ptr(cudaEventBlockingSync);
        if (E == nullptr) { S->detach(); S = nullptr; fail(de::DECX_FAIL_CUDA_EVENT, "error: Fail to access cuda event"); return false; }
        return true;
    }
    void wait() { E->event_record(S); E->synchronize(); }
    ~StreamEvent() { if (S) S->detach(); if (E) E->detach(); }
};

struct DeviceBlock {      // scratch from the device pool, returned on scope exit
    decx::PtrInfo<void> p;
    bool take(uint64_t bytes) { return bytes == 0 || decx::alloc::_device_malloc(&p, bytes) == 0; }
    ~DeviceBlock() { decx::alloc::_device_dealloc(&p); }
};

// trans: Vector x Matrix (reduce over the rows of the matrix)
void gemv_host(decx::_Vector* vec, decx::_Matrix* mat, decx::_Vector* dst, bool trans, uint32_t accu) {
    if (!decx::cuda::_is_CUDA_init()) return fail(de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first");
    if (vec == nullptr || mat == nullptr || dst == nullptr || !vec->_init || !mat->_init)
        return fail(de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    if (vec->Type() != mat->Type()) return fail(de::DECX_FAIL_TYPE_MOT_MATCH, "error: The types of the two objects are not equal");
    const de::_DATA_TYPES_FLAGS_ t = mat->Type();
    if (t != de::_FP32_ && t != de::_FP16_)
        return fail(de::DECX_FAIL_UNSUPPORTED_TYPE, "error: The data type is not supported by the matrix-vector product");
    if (t == de::_FP16_ && accu > de::Fp16_Accurate_L3) return fail(de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
    const uint32_t rows = mat->Height(), cols = mat->Width();
    if (vec->Len() != (trans ? rows : cols)) return fail(de::DECX_FAIL_DimsNotMatching, "error: Dim(s) is(are) not equal to each other");
    if (dst == vec) return fail(de::DECX_FAIL_INVALID_PARAM, "error: dst must not be one of the factors");
    const de::_DATA_TYPES_FLAGS_ out_t = (t == de::_FP32_ || accu == de::Fp16_Accurate_L1) ? de::_FP32_ : de::_FP16_;
    const uint64_t out_len = trans ? cols : rows;
    dst->re_construct(out_t, out_len);
    if (!dst->_init) return fail(de::DECX_FAIL_ALLOCATION, "error: Fail to allocate memory on RAM");

    const int dt = (t == de::_FP32_) ? DECXB200_FP32 : DECXB200_FP16;
    const uint64_t es = uint64_t(decx::element_size(t)), oes = uint64_t(decx::element_size(out_t));
    const uint64_t lda = decx::pitch_for(cols, int(es), 128);                       // the device-matrix pitch rule
    const size_t ws = decxb200_gemv_workspace_bytes(dt, int(accu), trans ? 1 : 0, rows, cols);
    DeviceBlock dA, dx, dy, dw;
    if (!dA.take(uint64_t(rows) * lda * es) || !dx.take(vec->total_bytes) || !dy.take((out_len + 8) * oes) || !dw.take(ws))
        return fail(de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
    StreamEvent se;
    if (!se.ok()) return;
    cudaStream_t s = se.S->get_raw_stream_ref();
    cudaError_t e = cudaMemcpy2DAsync(dA.p.ptr, lda * es, mat->data, uint64_t(mat->Pitch()) * es, uint64_t(cols) * es, rows,
                                      cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dx.p.ptr, vec->data, vec->Len() * es, cudaMemcpyHostToDevice, s);
    int rc = 0;
    if (e == cudaSuccess)
        rc = decxb200_gemv(dt, int(accu), trans ? 1 : 0, s, rows, cols, dA.p.ptr, lda, dx.p.ptr, dy.p.ptr, dw.p.ptr, ws);
    if (e == cudaSuccess && rc == 0) e = cudaMemcpyAsync(dst->data, dy.p.ptr, out_len * oes, cudaMemcpyDeviceToHost, s);
    se.wait();
    if (e != cudaSuccess) { cudaGetLastError(); return fail(de::DECX_FAIL_CUDA_STREAM, cudaGetErrorString(e)); }
    if (rc != 0) return fail(rc < 0 ? de::DECX_FAIL_INVALID_PARAM : de::DECX_FAIL_CUDA_STREAM, decxb200_strerror(rc));
}

}  // namespace

void de::blas::cuda::GEMM(de::Vector& A, de::Matrix& B, de::Vector& dst, const uint32_t _fp16_accu) {
    de::ResetLastError();
    gemv_host(dynamic_cast<decx::_Vector*>(&A), dynamic_cast<decx::_Matrix*>(&B), dynamic_cast<decx::_Vector*>(&dst), true,
              _fp16_accu);
}

void de::blas::cuda::GEMM(de::Matrix& A, de::Vector& B, de::Vector& dst, const uint32_t _fp16_accu) {
    de::ResetLastError();
    gemv_host(dynamic_cast<decx::_Vector*>(&B), dynamic_cast<decx::_Matrix*>(&A), dynamic_cast<decx::_Vector*>(&dst), false,
              _fp16_accu);
}

de::DH de::cuda::Transpose(de::GPU_Matrix& src, de::GPU_Matrix& dst) {
    de::ResetLastError();
    auto done = [] { return *de::GetLastError(); };
    if (!decx::cuda::_is_CUDA_init()) { fail(de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first"); return done(); }
    decx::_GPU_Matrix* s = dynamic_cast<decx::_GPU_Matrix*>(&src);
    decx::_GPU_Matrix* d = dynamic_cast<decx::_GPU_Matrix*>(&dst);
    if (s == nullptr || d == nullptr || !s->_init) { fail(de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized"); return done(); }
    if (s == d) { fail(de::DECX_FAIL_INVALID_PARAM, "error: dst must not be src"); return done(); }
    int prev = 0;
    cudaGetDevice(&prev);
    if (s->_device >= 0 && s->_device != prev) cudaSetDevice(s->_device);
    {
        StreamEvent se;
        if (se.ok()) {
            d->re_construct(s->Type(), s->Height(), s->Width(), se.S);           // (type, width, height)
            if (!d->_init) {
                fail(de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
            } else {
                const int rc = decxb200_transpose(s->_layout._single_element_size, se.S->get_raw_stream_ref(), s->Height(),
                                                  s->Width(), s->Mat.ptr, s->Pitch(), d->Mat.ptr, d->Pitch());
                se.wait();
                if (rc != 0) fail(rc < 0 ? de::DECX_FAIL_INVALID_PARAM : de::DECX_FAIL_CUDA_STREAM, decxb200_strerror(rc));
            }
        }
    }
    if (s->_device >= 0 && s->_device != prev) cudaSetDevice(prev);
    return done();
}

de::DH de::cuda::TypeCast(de::GPU_Matrix& src, de::GPU_Matrix& dst, const int cvt_method) {
    de::DH h;
    decx::err::success(&h);
    auto bad = [&](int code, const char* msg) { decx::err::set(&h, code, msg); decx::err::set(de::GetLastError(), code, msg); return h; };
    if (!decx::cuda::_is_CUDA_init()) return bad(de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first");
    decx::_GPU_Matrix* s = dynamic_cast<decx::_GPU_Matrix*>(&src);
    decx::_GPU_Matrix* d = dynamic_cast<decx::_GPU_Matrix*>(&dst);
    if (s == nullptr || d == nullptr || !s->_init) return bad(de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    if (s == d) return bad(de::DECX_FAIL_INVALID_PARAM, "error: dst must not be src");
    int kind;
    de::_DATA_TYPES_FLAGS_ from, to;
    switch (cvt_method) {
        case de::CVT_FP32_FP64: kind = DECXB200_CAST_F32_F64; from = de::_FP32_; to = de::_FP64_; break;
        case de::CVT_FP64_FP32: kind = DECXB200_CAST_F64_F32; from = de::_FP64_; to = de::_FP32_; break;
        case de::CVT_INT32_FP32: kind = DECXB200_CAST_I32_F32; from = de::_INT32_; to = de::_FP32_; break;
        case de::CVT_FP32_INT32: kind = DECXB200_CAST_F32_I32; from = de::_FP32_; to = de::_INT32_; break;
        case de::CVT_FP32_FP16: kind = DECXB200_CAST_F32_F16; from = de::_FP32_; to = de::_FP16_; break;
        case de::CVT_FP16_FP32: kind = DECXB200_CAST_F16_F32; from = de::_FP16_; to = de::_FP32_; break;
        default: return bad(de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
    }
    if (s->Type() != from) return bad(de::DECX_FAIL_TYPE_MOT_MATCH, "error: The source does not have the type this cast converts from");
    int prev = 0;
    cudaGetDevice(&prev);
    if (s->_device >= 0 && s->_device != prev) cudaSetDevice(s->_device);
    {
        StreamEvent se;
        if (!se.ok()) {
            h = *de::GetLastError();
        } else {
            d->re_construct(to, s->Width(), s->Height(), se.S);
            if (!d->_init) {
                bad(de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
            } else {
                const int rc = decxb200_cast2d(kind, se.S->get_raw_stream_ref(), s->Height(), s->Width(), s->Mat.ptr, s->Pitch(),
                                               d->Mat.ptr, d->Pitch());
                se.wait();
                if (rc != 0) bad(rc < 0 ? de::DECX_FAIL_INVALID_PARAM : de::DECX_FAIL_CUDA_STREAM, decxb200_strerror(rc));
            }
        }
    }
    if (s->_device >= 0 && s->_device != prev) cudaSetDevice(prev);
    return h;
}
