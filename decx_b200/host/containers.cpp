// Concrete host and device matrices and their factories: see internal.h for the reference citations.
#include <cstdlib>
#include <cstring>

#include <cstdio>
#include <cstdlib>
#if defined(__linux__)
#include <sys/syscall.h>
#include <unistd.h>
#endif

#include "internal.h"

// ------------------------------------------------------------------------------------------------ host matrix
namespace {
// Host matrices of 64 MiB and more get their pages interleaved over the NUMA nodes of the machine (mbind,
// MPOL_INTERLEAVE, before the first touch).  A matrix that one thread allocates and zero-fills would otherwise live
// on that thread's node alone, so every GPU behind the other socket would pull its rows across the inter-socket
// link when all GPUs move their row blocks at once.  A precaution: on the eight-GPU machine this was measured on,
// the aggregate host-to-device rate was the same with and without it.  Best effort: any failure leaves the default
// placement.
void interleave_pages(void* addr, uint64_t bytes) {
#if defined(__linux__) && defined(SYS_mbind)
    unsigned long mask = 0;
    if (FILE* f = std::fopen("/sys/devices/system/node/online", "r")) {
        char buf[128] = {0};
        if (std::fgets(buf, sizeof(buf), f) != nullptr) {
            for (const char* p = buf; *p != '\0' && *p != '\n';) {          // "0-1", "0,2-3", ...
                char* end = nullptr;
                const long a = std::strtol(p, &end, 10);
                if (end == p) break;
                long b = a;
                p = end;
                if (*p == '-') { b = std::strtol(p + 1, &end, 10); p = end; }
                for (long n = a; n <= b && n < 64; ++n) mask |= 1ul << n;
                if (*p == ',') ++p;
            }
        }
        std::fclose(f);
    }
    if ((mask & (mask - 1)) == 0) return;                                  // one node (or none known): nothing to spread
    const int MPOL_INTERLEAVE_ = 3;
    syscall(SYS_mbind, addr, static_cast<unsigned long>(bytes), MPOL_INTERLEAVE_, &mask, 65ul, 0u);
#else
    (void)addr; (void)bytes;
#endif
}
}  // namespace

namespace {
void fill_layout(de::MatrixLayout& l, de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t align_bytes) {
    l._single_element_size = decx::element_size(t);
    l.width = w;
    l.height = h;
    l.pitch = decx::pitch_for(w, l._single_element_size, align_bytes);
}
}  // namespace

decx::_Matrix::_Matrix() {
    std::memset(&_layout, 0, sizeof(_layout));
    this->_exp_data_ptr = &this->data;
    this->_exp_matrix_dscr = &this->_layout;
}

decx::_Matrix::_Matrix(const de::_DATA_TYPES_FLAGS_ t, const uint32_t width, const uint32_t height,
                       const de::_DATA_FORMATS_ format) : _Matrix() {
    construct(t, width, height, format);
}

void decx::_Matrix::construct(const de::_DATA_TYPES_FLAGS_ t, uint32_t width, uint32_t height,
                              const de::_DATA_FORMATS_ format) {
    release();
    type = t;
    _format = format;
    fill_layout(_layout, t, width, height, 32);      // host rows start 32 bytes apart or more (Matrix.cxx:35-64)
    total_bytes = uint64_t(_layout.pitch) * height * _layout._single_element_size;
    if (total_bytes == 0) return;
    const uint64_t padded = (total_bytes + 63) / 64 * 64;
    // large matrices are page-aligned so that their pages can be spread over the NUMA nodes before first touch
    data = std::aligned_alloc(padded >= (64u << 20) ? 4096 : 64, padded >= (64u << 20) ? (padded + 4095) / 4096 * 4096 : padded);
    if (data == nullptr) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_ALLOCATION, "error: Fail to allocate memory on RAM");
        return;
    }
    if (padded >= (64u << 20)) interleave_pages(data, (padded + 4095) / 4096 * 4096);
    std::memset(data, 0, padded);
    _shared = new int(1);
    _owner = true;
    _init = true;
}

void decx::_Matrix::re_construct(const de::_DATA_TYPES_FLAGS_ t, uint32_t width, uint32_t height) {
    if (_init && t == type && width == _layout.width && height == _layout.height) return;
    const uint64_t need = uint64_t(decx::pitch_for(width, decx::element_size(t), 32)) * height * decx::element_size(t);
    if (_init && need <= total_bytes && _shared != nullptr && *_shared == 1) {   // fits: keep the storage
        const uint64_t cap = total_bytes;
        type = t;
        fill_layout(_layout, t, width, height, 32);
        total_bytes = cap;
        return;
    }
    construct(t, width, height, _format);
}

uint32_t decx::_Matrix::Width() const { return _layout.width; }
uint32_t decx::_Matrix::Height() const { return _layout.height; }
de::_DATA_TYPES_FLAGS_ decx::_Matrix::Type() const { return type; }
de::_DATA_FORMATS_ decx::_Matrix::Format() const { return _format; }

void decx::_Matrix::release() {
    if (data != nullptr && _shared != nullptr && --(*_shared) == 0) {
        if (_pinned) cudaHostUnregister(data);
        std::free(data);
        delete _shared;
    }
    data = nullptr;
    _shared = nullptr;
    _pinned = false;
    _init = false;
    total_bytes = 0;
}

// shares src's storage (reference: Matrix.cxx "SoftCopy": same block, one more reference)
de::Matrix& decx::_Matrix::SoftCopy(de::Matrix& src) {
    decx::_Matrix& s = dynamic_cast<decx::_Matrix&>(src);
    if (&s == this) return *this;
    release();
    _layout = s._layout;
    type = s.type;
    _format = s._format;
    total_bytes = s.total_bytes;
    data = s.data;
    _shared = s._shared;
    _pinned = s._pinned;
    if (_shared != nullptr) ++(*_shared);
    _init = s._init;
    return *this;
}

// same bytes, another element type of the same row size (e.g. cplxf <-> 2 x fp32 per element)
void decx::_Matrix::Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) {
    const int ns = decx::element_size(_new_type);
    if (ns == 0 || !_init) return;
    const uint64_t row_bytes = uint64_t(_layout.pitch) * _layout._single_element_size;
    const uint64_t width_bytes = uint64_t(_layout.width) * _layout._single_element_size;
    if (row_bytes % ns != 0 || width_bytes % ns != 0) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
        return;
    }
    type = _new_type;
    _layout._single_element_size = ns;
    _layout.pitch = uint32_t(row_bytes / ns);
    _layout.width = uint32_t(width_bytes / ns);
}

decx::_Matrix::~_Matrix() { release(); }

de::Matrix* de::CreateMatrixPtr() { return new decx::_Matrix(); }
de::Matrix& de::CreateMatrixRef() { return *(new decx::_Matrix()); }
de::Matrix* de::CreateMatrixPtr(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width, const uint32_t _height,
                                const de::_DATA_FORMATS_ format) {
    return new decx::_Matrix(type, _width, _height, format);
}
de::Matrix& de::CreateMatrixRef(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width, const uint32_t _height,
                                const de::_DATA_FORMATS_ format) {
    return *(new decx::_Matrix(type, _width, _height, format));
}

de::DH de::cuda::PinMemory(de::Matrix& src) {
    de::DH h;
    decx::err::success(&h);
    decx::_Matrix* m = dynamic_cast<decx::_Matrix*>(&src);
    if (m == nullptr || !m->_init) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (m->_pinned) {
        decx::err::set(&h, de::DECX_FAIL_HOST_MEM_REGISTERED, "error: The host memory is already registered");
    } else if (cudaHostRegister(m->data, (m->total_bytes + 63) / 64 * 64, cudaHostRegisterPortable) != cudaSuccess) {
        cudaGetLastError();
        decx::err::set(&h, de::DECX_FAIL_ALLOCATION, "error: Fail to register the host memory");
    } else {
        m->_pinned = true;
    }
    return h;
}

de::DH de::cuda::UnpinMemory(de::Matrix& src) {
    de::DH h;
    decx::err::success(&h);
    decx::_Matrix* m = dynamic_cast<decx::_Matrix*>(&src);
    if (m == nullptr || !m->_init) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (!m->_pinned) {
        decx::err::set(&h, de::DECX_FAIL_HOST_MEM_UNREGISTERED, "error: The host memory is not registered");
    } else {
        cudaHostUnregister(m->data);
        m->_pinned = false;
    }
    return h;
}

// ------------------------------------------------------------------------------------------------ device matrix
decx::_GPU_Matrix::_GPU_Matrix() { std::memset(&_layout, 0, sizeof(_layout)); }

decx::_GPU_Matrix::_GPU_Matrix(const de::_DATA_TYPES_FLAGS_ t, const uint32_t width, const uint32_t height,
                               const de::_DATA_FORMATS_ format) : _GPU_Matrix() {
    construct(t, width, height, format);
}

void decx::_GPU_Matrix::construct(const de::_DATA_TYPES_FLAGS_ t, uint32_t width, uint32_t height,
                                  const de::_DATA_FORMATS_ format) {
    release();
    type = t;
    _format = format;
    fill_layout(_layout, t, width, height, 128);     // device rows start 128 bytes apart or more (GPU_Matrix.cu:35-61)
    total_bytes = uint64_t(_layout.pitch) * height * _layout._single_element_size;
    if (total_bytes == 0) return;
    cudaGetDevice(&_device);
    // zero-filled like the reference (GPU_Matrix.cu:65-96): GEMM never relies on it, user code may
    if (decx::alloc::_device_malloc(&Mat, total_bytes, true, nullptr) != 0) {
        cudaGetLastError();
        decx::err::set(de::GetLastError(), de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
        total_bytes = 0;
        return;
    }
    _init = true;
}

void decx::_GPU_Matrix::re_construct(const de::_DATA_TYPES_FLAGS_ t, uint32_t width, uint32_t height,
                                     decx::cuda_stream* S) {
    // a block is only kept if it lives in the pool of the device that is current now (the device the caller
    // is about to launch on) and the pool has not been released under it
    int now_dev = 0;
    cudaGetDevice(&now_dev);
    const bool usable = Mat.block != nullptr && !Mat.block->orphan &&
                        Mat.block->pool == decx::MemPool_D::GetInstance(now_dev);
    if (_init && usable && t == type && width == _layout.width && height == _layout.height) return;
    const int es = decx::element_size(t);
    const uint64_t need = uint64_t(decx::pitch_for(width, es, 128)) * height * es;
    type = t;
    fill_layout(_layout, t, width, height, 128);
    if (_init && usable && Mat.block->size >= need && Mat.block->refcount == 1) {
        total_bytes = need;                           // grow-only: the block is kept
        return;
    }
    if (Mat.block != nullptr) {
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur != _device && _device >= 0) cudaSetDevice(_device);
        decx::alloc::_device_dealloc(&Mat);
        if (cur != _device && _device >= 0) cudaSetDevice(cur);
    }
    _init = false;
    total_bytes = need;
    if (need == 0) return;
    cudaGetDevice(&_device);
    if (decx::alloc::_device_malloc(&Mat, need, true, S) != 0) {
        cudaGetLastError();
        decx::err::set(de::GetLastError(), de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
        total_bytes = 0;
        return;
    }
    _init = true;
}

uint decx::_GPU_Matrix::Width() const { return _layout.width; }
uint decx::_GPU_Matrix::Height() const { return _layout.height; }
de::_DATA_TYPES_FLAGS_ decx::_GPU_Matrix::Type() const { return type; }
de::_DATA_FORMATS_ decx::_GPU_Matrix::Format() const { return _format; }

void decx::_GPU_Matrix::release() {
    if (Mat.block != nullptr) {
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur != _device && _device >= 0) cudaSetDevice(_device);
        decx::alloc::_device_dealloc(&Mat);
        if (cur != _device && _device >= 0) cudaSetDevice(cur);
    }
    _init = false;
    total_bytes = 0;
}

de::GPU_Matrix& decx::_GPU_Matrix::SoftCopy(de::GPU_Matrix& src) {
    decx::_GPU_Matrix& s = dynamic_cast<decx::_GPU_Matrix&>(src);
    if (&s == this) return *this;
    release();
    _layout = s._layout;
    type = s.type;
    _format = s._format;
    total_bytes = s.total_bytes;
    _device = s._device;
    Mat = s.Mat;
    if (Mat.block != nullptr) {
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur != _device && _device >= 0) cudaSetDevice(_device);
        decx::alloc::_device_malloc_same_place(&Mat);
        if (cur != _device && _device >= 0) cudaSetDevice(cur);
    }
    _init = s._init;
    return *this;
}

void decx::_GPU_Matrix::Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) {
    const int ns = decx::element_size(_new_type);
    if (ns == 0 || !_init) return;
    const uint64_t row_bytes = uint64_t(_layout.pitch) * _layout._single_element_size;
    const uint64_t width_bytes = uint64_t(_layout.width) * _layout._single_element_size;
    if (row_bytes % ns != 0 || width_bytes % ns != 0) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
        return;
    }
    type = _new_type;
    _layout._single_element_size = ns;
    _layout.pitch = uint32_t(row_bytes / ns);
    _layout.width = uint32_t(width_bytes / ns);
}

// like the reference, the destructor of a device matrix does not return its block (GPU_Matrix.cu); call release()
decx::_GPU_Matrix::~_GPU_Matrix() {}

de::GPU_Matrix& de::CreateGPUMatrixRef() { return *(new decx::_GPU_Matrix()); }
de::GPU_Matrix* de::CreateGPUMatrixPtr() { return new decx::_GPU_Matrix(); }
de::GPU_Matrix* de::CreateGPUMatrixPtr(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width, const uint32_t _height,
                                       const de::_DATA_FORMATS_ format) {
    return new decx::_GPU_Matrix(type, _width, _height, format);
}
de::GPU_Matrix& de::CreateGPUMatrixRef(const de::_DATA_TYPES_FLAGS_ type, const uint32_t _width, const uint32_t _height,
                                       const de::_DATA_FORMATS_ format) {
    return *(new decx::_GPU_Matrix(type, _width, _height, format));
}

// ------------------------------------------------------------------------------------------------ de::Memcpy
// (reference: srcs/modules/core/data transmission/data_transmission.cu:105-180)
de::DH de::Memcpy(de::Matrix& __host, de::GPU_Matrix& __device, const de::Point2D start_src, de::Point2D start_dst,
                  const de::Point2D cpy_size, const int _memcpy_flag) {
    de::DH h;
    decx::err::success(&h);
    if (!decx::cuda::_is_CUDA_init()) {
        decx::err::set(&h, de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first");
        decx::err::set(de::GetLastError(), h.error_type, h.error_string);
        return h;
    }
    decx::_Matrix* hm = dynamic_cast<decx::_Matrix*>(&__host);
    decx::_GPU_Matrix* dm = dynamic_cast<decx::_GPU_Matrix*>(&__device);
    if (hm == nullptr || dm == nullptr || !hm->_init || !dm->_init) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (hm->type != dm->type) {
        decx::err::set(&h, de::MEMCPY_DIFFERENT_TYPES, "error: The types of the two objects are not equal");
    } else {
        const bool h2d = (_memcpy_flag == de::DECX_MEMCPY_H2D);
        const uint32_t sw = h2d ? hm->Width() : dm->Width(), sh = h2d ? hm->Height() : dm->Height();
        const uint32_t dw = h2d ? dm->Width() : hm->Width(), dh = h2d ? dm->Height() : hm->Height();
        if (_memcpy_flag != de::DECX_MEMCPY_H2D && _memcpy_flag != de::DECX_MEMCPY_D2H) {
            decx::err::set(&h, de::DECX_FAIL_ErrorFlag, "error: This flag is meaningless in current context");
        } else if (start_src.x < 0 || start_src.y < 0 || start_dst.x < 0 || start_dst.y < 0 || cpy_size.x < 0 ||
                   cpy_size.y < 0 || uint64_t(start_src.x) + cpy_size.x > sw || uint64_t(start_src.y) + cpy_size.y > sh ||
                   uint64_t(start_dst.x) + cpy_size.x > dw || uint64_t(start_dst.y) + cpy_size.y > dh) {
            decx::err::set(&h, de::DECX_FAIL_MEMCPY_OVERRANGED, "error: The copy area exceeds the matrix");
        } else if (cpy_size.x > 0 && cpy_size.y > 0) {
            const uint64_t es = uint64_t(hm->_layout._single_element_size);
            uint8_t* hp = static_cast<uint8_t*>(hm->data);
            uint8_t* dp = static_cast<uint8_t*>(dm->Mat.ptr);
            const uint64_t hpitch = hm->Pitch() * es, dpitch = dm->Pitch() * es;
            cudaError_t e;
            if (h2d)
                e = cudaMemcpy2D(dp + start_dst.y * dpitch + start_dst.x * es, dpitch,
                                 hp + start_src.y * hpitch + start_src.x * es, hpitch, cpy_size.x * es, cpy_size.y,
                                 cudaMemcpyHostToDevice);
            else
                e = cudaMemcpy2D(hp + start_dst.y * hpitch + start_dst.x * es, hpitch,
                                 dp + start_src.y * dpitch + start_src.x * es, dpitch, cpy_size.x * es, cpy_size.y,
                                 cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) {
                cudaGetLastError();
                decx::err::set(&h, de::DECX_FAIL_CUDA_STREAM, cudaGetErrorString(e));
            }
        }
    }
    if (h.error_type != de::DECX_SUCCESS) decx::err::set(de::GetLastError(), h.error_type, h.error_string);
    return h;
}
