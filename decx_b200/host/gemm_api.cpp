// de::blas::cuda::GEMM -- the four overloads of the drop-in.
//
// Reference flow (srcs/modules/BLAS/GEMM/CUDA/GEMM_LS.cu:62-109, 315-393): cast to the concrete matrices,
// validate, take a pooled non-blocking stream and a blocking-sync event, re-construct dst, plan, launch the
// chosen SIMT kernel, record + wait on the event, give stream and event back.  This file keeps that flow and
// its error codes; "plan + launch" is one call into the C ABI (include/decx_b200.h), and the planner-owned
// A-transpose scratch is replaced by the tf32-plane workspace, cached with the reference's 5 s lifespan.
// Unlike the reference, a failed validation returns before anything is launched, and nothing calls exit().
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/decx_b200.h"
#include "internal.h"

namespace {

int abi_dtype(de::_DATA_TYPES_FLAGS_ t) {
    switch (t) {
        case de::_FP32_: return DECXB200_FP32;
        case de::_FP16_: return DECXB200_FP16;
        case de::_COMPLEX_F32_: return DECXB200_CPLXF;
        case de::_FP64_: return DECXB200_FP64;
        case de::_COMPLEX_F64_: return DECXB200_CPLXD;
        default: return -1;
    }
}

void fail(int code, const char* msg) { decx::err::set(de::GetLastError(), code, msg); }

// alpha / beta as the accumulate type the C ABI wants: float / {re, im} floats for the 16/32-bit types, double /
// {re, im} doubles for fp64 and complex fp64 (the same 16 bytes hold either)
union AbiScalar {
    float f[2];
    double d[2];
};
bool scalar_of(const de::Number& n, de::_DATA_TYPES_FLAGS_ t, AbiScalar& out) {
    if (n.Type() != int32_t(t)) return false;
    if (t == de::_FP64_) { out.d[0] = n.get_data_ref<double>(); out.d[1] = 0.0; return true; }
    if (t == de::_COMPLEX_F64_) { out.d[0] = n.get_data_ref<de::CPd>().real; out.d[1] = n.get_data_ref<de::CPd>().image; return true; }
    out.f[1] = 0.f;
    if (t == de::_FP32_) out.f[0] = n.get_data_ref<float>();
    else if (t == de::_FP16_) out.f[0] = de::Half2Float(n.get_data_ref<de::Half>());
    else {
        out.f[0] = n.get_data_ref<de::CPf>().real;
        out.f[1] = n.get_data_ref<de::CPf>().image;
    }
    return true;
}

void report_abi_error(int rc) {
    if (rc == DECXB200_EALIGN || rc == DECXB200_EINVAL || rc == DECXB200_ETOOLARGE)
        fail(de::DECX_FAIL_INVALID_PARAM, decxb200_strerror(rc));
    else if (rc == DECXB200_EWORKSPACE)
        fail(de::DECX_FAIL_CUDA_ALLOCATION, decxb200_strerror(rc));
    else if (rc == DECXB200_EDRIVER)
        fail(de::DECX_FAIL_CUDA_not_init, decxb200_strerror(rc));
    else
        fail(de::DECX_FAIL_CUDA_STREAM, decxb200_strerror(rc));
}

// scratch caches, created on first use and never destroyed (like the reference's planners they are owned by
// the resource manager, which returns their memory after 5 idle seconds)
decx::ScratchResource* arena_cache() {
    static decx::ScratchResource* r = new decx::ScratchResource(5.0);
    return r;
}
// below this much arithmetic one GPU finishes before several could be set up (DECX_B200_MULTI_MIN_FLOPS overrides)
double multi_min_flops() {
    const char* e = getenv("DECX_B200_MULTI_MIN_FLOPS");
    const double v = e ? atof(e) : 0.0;
    return v > 0.0 ? v : 4.0e12;
}
decx::ScratchResource* multi_arena_cache(int device) {          // one per device for the multi-GPU host path
    static std::mutex mtx;
    static decx::ScratchResource* r[64] = {nullptr};
    std::lock_guard<std::mutex> lk(mtx);
    if (r[device & 63] == nullptr) r[device & 63] = new decx::ScratchResource(5.0);
    return r[device & 63];
}

// Status words for the kernels' bounded waits: 64 slots per device (device words straight from cudaMalloc, so they
// outlive a release of the pool, and a pinned host mirror to read them back).  Every call takes a slot of its own,
// so calls from several host threads do not share state; a 65th concurrent call waits for a slot.
struct StatusSlots {
    unsigned* dev = nullptr;
    unsigned* host = nullptr;
    uint64_t used = 0;
    std::mutex mtx;
    std::condition_variable cv;
};
StatusSlots* status_slots(int device) {
    static std::mutex mtx;
    static StatusSlots slots[64];
    if (device < 0 || device >= 64) return nullptr;
    StatusSlots& w = slots[device];
    std::lock_guard<std::mutex> lk(mtx);
    if (w.dev == nullptr) {
        void* d = nullptr;
        if (cudaMalloc(&d, 64 * sizeof(unsigned)) != cudaSuccess || cudaMemset(d, 0, 64 * sizeof(unsigned)) != cudaSuccess) {
            cudaGetLastError();
            if (d != nullptr) cudaFree(d);
            return nullptr;
        }
        if (cudaHostAlloc(reinterpret_cast<void**>(&w.host), 64 * sizeof(unsigned), cudaHostAllocDefault) != cudaSuccess) {
            cudaGetLastError();
            cudaFree(d);
            return nullptr;
        }
        std::memset(w.host, 0, 64 * sizeof(unsigned));
        w.dev = static_cast<unsigned*>(d);
    }
    return &w;
}
struct StatusWord {            // one slot, held for the duration of a call
    StatusSlots* owner = nullptr;
    int index = -1;
    unsigned* dev() const { return owner->dev + index; }
    unsigned* host() const { return owner->host + index; }
    bool take(int device) {
        owner = status_slots(device);
        if (owner == nullptr) return false;
        std::unique_lock<std::mutex> lk(owner->mtx);
        owner->cv.wait(lk, [&] { return owner->used != ~0ull; });
        for (int i = 0; i < 64; ++i)
            if (!(owner->used >> i & 1ull)) { owner->used |= 1ull << i; index = i; break; }
        return true;
    }
    ~StatusWord() {
        if (owner == nullptr || index < 0) return;
        {
            std::lock_guard<std::mutex> lk(owner->mtx);
            owner->used &= ~(1ull << index);
        }
        owner->cv.notify_one();
    }
};

struct DeviceScope {   // makes `device` current for the call, restores the caller's device afterwards
    int prev = 0;
    bool switched = false;
    explicit DeviceScope(int device) {
        cudaGetDevice(&prev);
        if (device >= 0 && device != prev) { cudaSetDevice(device); switched = true; }
    }
    ~DeviceScope() { if (switched) cudaSetDevice(prev); }
};

void gemm_device(de::GPU_Matrix& A_, de::GPU_Matrix& B_, de::GPU_Matrix* C_, de::GPU_Matrix& dst_,
                 const de::Number* alpha, const de::Number* beta) {
    decx::_GPU_Matrix* A = dynamic_cast<decx::_GPU_Matrix*>(&A_);
    decx::_GPU_Matrix* B = dynamic_cast<decx::_GPU_Matrix*>(&B_);
    decx::_GPU_Matrix* C = C_ ? dynamic_cast<decx::_GPU_Matrix*>(C_) : nullptr;
    decx::_GPU_Matrix* dst = dynamic_cast<decx::_GPU_Matrix*>(&dst_);
    if (!decx::cuda::_is_CUDA_init()) return fail(de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first");
    if (A == nullptr || B == nullptr || dst == nullptr || (C_ && C == nullptr) || !A->_init || !B->_init || (C && !C->_init))
        return fail(de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    // validation of the reference (large_squares/common/cuda_GEMM_LS_planner.cu:229-258) plus C's extents,
    // which its CUDA path forgets and its CPU path checks (cpu_GEMM_config.cxx:218-224)
    if (A->Width() != B->Height()) return fail(de::DECX_FAIL_DimsNotMatching, "error: Dim(s) is(are) not equal to each other");
    if (A->Type() != B->Type() || (C && C->Type() != A->Type()))
        return fail(de::DECX_FAIL_TYPE_MOT_MATCH, "error: The types of the two objects are not equal");
    const int dt = abi_dtype(A->Type());
    if (dt < 0) return fail(de::DECX_FAIL_UNSUPPORTED_TYPE, "error: The data type is not supported by GEMM on this path");
    if (C && (C->Width() != B->Width() || C->Height() != A->Height()))
        return fail(de::DECX_FAIL_DimsNotMatching, "error: Dim(s) is(are) not equal to each other");
    AbiScalar a, b;
    if (C) {
        if (!scalar_of(*alpha, A->Type(), a) || !scalar_of(*beta, A->Type(), b))
            return fail(de::DECX_FAIL_TYPE_MOT_MATCH, "error: The types of the two objects are not equal");
    }
    if (dst == A || dst == B) return fail(de::DECX_FAIL_INVALID_PARAM, "error: dst must not be one of the factors");
    if (B->_device != A->_device || (C && C->_device != A->_device))
        return fail(de::DECX_FAIL_INVALID_PARAM, "error: the matrices live on different devices");

    DeviceScope scope(A->_device);
    decx::cuda_stream* S = decx::cuda::get_cuda_stream_ptr(cudaStreamNonBlocking);
    if (S == nullptr) return fail(de::DECX_FAIL_CUDA_STREAM, "error: Fail to access cuda stream");
    decx::cuda_event* E = decx::cuda::get_cuda_event_ptr(cudaEventBlockingSync);
    if (E == nullptr) {
        S->detach();
        return fail(de::DECX_FAIL_CUDA_EVENT, "error: Fail to access cuda event");
    }
    const uint32_t M = A->Height(), N = B->Width(), K = A->Width();
    dst->re_construct(A->Type(), N, M, S);
    StatusWord sw;
    if (!dst->_init || !sw.take(A->_device)) {
        S->detach();
        E->detach();
        return fail(de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
    }
    // scratch of THIS call, from the device pool (carved out of chunks the pool already holds after the first
    // calls): concurrent calls from several host threads each have their own and run on their own streams
    const size_t need = decxb200_gemm_workspace_bytes(dt, M, N, K);
    decx::PtrInfo<void> ws;
    if (need && decx::alloc::_device_malloc(&ws, need) != 0) {
        cudaGetLastError();
        S->detach();
        E->detach();
        return fail(de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
    }
    const int rc = decxb200_gemm(dt, S->get_raw_stream_ref(), M, N, K, A->Mat.ptr, A->Pitch(), B->Mat.ptr, B->Pitch(),
                                 C ? C->Mat.ptr : nullptr, C ? C->Pitch() : 0, dst->Mat.ptr, dst->Pitch(), C ? &a : nullptr,
                                 C ? &b : nullptr, ws.ptr, need, sw.dev());
    if (rc == 0)
        cudaMemcpyAsync(sw.host(), sw.dev(), sizeof(unsigned), cudaMemcpyDeviceToHost, S->get_raw_stream_ref());
    E->event_record(S);
    E->synchronize();                       // the API is synchronous, as in the reference (GEMM_LS.cu:102-103)
    decx::alloc::_device_dealloc(&ws);
    S->detach();
    E->detach();
    if (rc != 0) return report_abi_error(rc);
    if (*sw.host() != 0) {
        char msg[96];
        snprintf(msg, sizeof(msg), "error: a bounded wait inside the GEMM kernel expired (code 0x%x)", *sw.host());
        *sw.host() = 0;
        cudaMemset(sw.dev(), 0, sizeof(unsigned));
        return fail(de::DECX_FAIL_CUDA_STREAM, msg);
    }
}

void gemm_host(de::Matrix& A_, de::Matrix& B_, de::Matrix* C_, de::Matrix& dst_) {
    decx::_Matrix* A = dynamic_cast<decx::_Matrix*>(&A_);
    decx::_Matrix* B = dynamic_cast<decx::_Matrix*>(&B_);
    decx::_Matrix* C = C_ ? dynamic_cast<decx::_Matrix*>(C_) : nullptr;
    decx::_Matrix* dst = dynamic_cast<decx::_Matrix*>(&dst_);
    if (!decx::cuda::_is_CUDA_init()) return fail(de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first");
    if (A == nullptr || B == nullptr || dst == nullptr || (C_ && C == nullptr) || !A->_init || !B->_init || (C && !C->_init))
        return fail(de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    if (A->Width() != B->Height()) return fail(de::DECX_FAIL_DimsNotMatching, "error: Dim(s) is(are) not equal to each other");
    if (A->Type() != B->Type() || (C && C->Type() != A->Type()))
        return fail(de::DECX_FAIL_TYPE_MOT_MATCH, "error: The types of the two objects are not equal");
    const int dt = abi_dtype(A->Type());
    if (dt < 0) return fail(de::DECX_FAIL_UNSUPPORTED_TYPE, "error: The data type is not supported by GEMM on this path");
    if (C && (C->Width() != B->Width() || C->Height() != A->Height()))
        return fail(de::DECX_FAIL_DimsNotMatching, "error: Dim(s) is(are) not equal to each other");
    if (dst == A || dst == B) return fail(de::DECX_FAIL_INVALID_PARAM, "error: dst must not be one of the factors");
    const uint32_t M = A->Height(), N = B->Width(), K = A->Width();
    dst->re_construct(A->Type(), N, M);
    if (!dst->_init) return fail(de::DECX_FAIL_ALLOCATION, "error: Fail to allocate memory on RAM");
    int device = 0;
    cudaGetDevice(&device);
    // Large fp16 products without a C operand are sharded by rows over every visible GPU: each GPU moves its rows
    // over its own PCIe link and the GPUs complete each other's copy of B over NVLink (decxb200_gemm_host_multi).
    // DECX_B200_MULTI_GPU=0 keeps the call on the current device; =N caps the number of GPUs used.
    if (dt == DECXB200_FP16 && C == nullptr && (N % 8) == 0) {
        static const int cap = [] { const char* e = getenv("DECX_B200_MULTI_GPU"); return e ? atoi(e) : 64; }();
        int ndev = 0;
        if (cap > 1 && cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 1 &&
            2.0 * double(M) * double(N) * double(K) >= multi_min_flops() && M >= 512) {
            if (ndev > cap) ndev = cap;
            if (ndev > 16) ndev = 16;
            const uint32_t tiles = (M + 255) / 256;
            if (uint32_t(ndev) > tiles) ndev = int(tiles);
            const size_t each = decxb200_gemm_host_multi_arena_bytes(dt, ndev, M, N, K);
            int devs[16];
            void* arenas[16];
            int got = 0;
            for (int d = 0; d < ndev; ++d) {
                devs[d] = (device + d) % ndev;                    // the caller's device first
                cudaSetDevice(devs[d]);
                arenas[d] = multi_arena_cache(devs[d])->lock(each, devs[d]);
                if (arenas[d] == nullptr) break;
                ++got;
            }
            cudaSetDevice(device);
            int rc = -1;
            if (got == ndev)
                rc = decxb200_gemm_host_multi(dt, ndev, devs, M, N, K, A->data, A->Pitch(), B->data, B->Pitch(), dst->data,
                                              dst->Pitch(), arenas, each);
            for (int d = 0; d < got; ++d) multi_arena_cache(devs[d])->unlock();
            if (got == ndev) {
                if (rc != 0) report_abi_error(rc);
                return;
            }
            cudaGetLastError();                                   // not enough memory somewhere: one GPU does it
        }
    }
    StatusWord sw;
    const bool have_sw = sw.take(device);
    const size_t need = decxb200_gemm_host_arena_bytes(dt, M, N, K, C ? 1 : 0);
    void* arena = arena_cache()->lock(need, device);
    if (arena == nullptr || !have_sw) {
        if (arena != nullptr) arena_cache()->unlock();
        return fail(de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
    }
    AbiScalar one;
    if (A->Type() == de::_FP64_ || A->Type() == de::_COMPLEX_F64_) { one.d[0] = 1.0; one.d[1] = 0.0; }
    else { one.f[0] = 1.f; one.f[1] = 0.f; }
    const int rc = decxb200_gemm_host(dt, M, N, K, A->data, A->Pitch(), B->data, B->Pitch(), C ? C->data : nullptr,
                                      C ? C->Pitch() : 0, dst->data, dst->Pitch(), C ? &one : nullptr, C ? &one : nullptr,
                                      arena, need, sw.dev());
    arena_cache()->unlock();
    if (rc == DECXB200_EKERNEL) {
        cudaMemset(sw.dev(), 0, sizeof(unsigned));
        return fail(de::DECX_FAIL_CUDA_STREAM, decxb200_strerror(rc));
    }
    if (rc != 0) return report_abi_error(rc);
}

}  // namespace

void de::blas::cuda::GEMM(de::GPU_Matrix& A, de::GPU_Matrix& B, de::GPU_Matrix& dst) {
    gemm_device(A, B, nullptr, dst, nullptr, nullptr);
}

void de::blas::cuda::GEMM(de::GPU_Matrix& A, de::GPU_Matrix& B, de::GPU_Matrix& C, de::GPU_Matrix& dst,
                          const de::Number alpha, const de::Number beta) {
    gemm_device(A, B, &C, dst, &alpha, &beta);
}

void de::blas::cuda::GEMM(de::Matrix& A, de::Matrix& B, de::Matrix& dst) { gemm_host(A, B, nullptr, dst); }

void de::blas::cuda::GEMM(de::Matrix& A, de::Matrix& B, de::Matrix& C, de::Matrix& dst) { gemm_host(A, B, &C, dst); }
