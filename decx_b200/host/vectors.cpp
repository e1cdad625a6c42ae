// de::Vector / de::GPU_Vector objects and their factories, pinning and de::Memcpy
// (reference: srcs/modules/core/classes/Vector.cxx, GPU_Vector.cu; srcs/modules/core/data transmission/
// data_transmission.cu:37-100).  Fresh implementations behind the reference's interfaces.
#include <cstdlib>
#include <cstring>

#include "internal.h"

namespace {
uint64_t padded(uint64_t n, uint64_t to) { return (n + to - 1) / to * to; }
}  // namespace

// ------------------------------------------------------------------------------------------------ host vector
decx::_Vector::_Vector() { _exp_data_ptr = &data; }
decx::_Vector::_Vector(const de::_DATA_TYPES_FLAGS_ t, uint64_t len) : _Vector() { construct(t, len); }

void decx::_Vector::construct(const de::_DATA_TYPES_FLAGS_ t, uint64_t len) {
    release();
    type = t;
    _single_element_size = decx::element_size(t);
    length = len;
    _length = padded(len, 8);
    total_bytes = _length * uint64_t(_single_element_size);
    if (total_bytes == 0) return;
    data = std::aligned_alloc(64, padded(total_bytes, 64));
    if (data == nullptr) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_ALLOCATION, "error: Fail to allocate memory on RAM");
        total_bytes = 0;
        return;
    }
    std::memset(data, 0, padded(total_bytes, 64));
    _shared = new int(1);
    _init = true;
}

void decx::_Vector::re_construct(const de::_DATA_TYPES_FLAGS_ t, uint64_t len) {
    if (_init && t == type && len == length) return;
    const uint64_t need = padded(len, 8) * uint64_t(decx::element_size(t));
    if (_init && _shared != nullptr && *_shared == 1 && need <= total_bytes && !_pinned) {
        type = t;                                   // grow-only: the storage is kept
        _single_element_size = decx::element_size(t);
        length = len;
        _length = padded(len, 8);
        return;
    }
    construct(t, len);
}

size_t decx::_Vector::Len() const { return length; }
de::_DATA_TYPES_FLAGS_ decx::_Vector::Type() const { return type; }

void decx::_Vector::release() {
    if (_shared != nullptr && --(*_shared) == 0) {
        if (_pinned) cudaHostUnregister(data);
        std::free(data);
        delete _shared;
    }
    _shared = nullptr;
    data = nullptr;
    _init = false;
    _pinned = false;
    total_bytes = 0;
    length = _length = 0;
}

de::Vector& decx::_Vector::SoftCopy(de::Vector& src) {
    decx::_Vector& s = dynamic_cast<decx::_Vector&>(src);
    if (&s == this) return *this;
    release();
    length = s.length; _length = s._length; total_bytes = s.total_bytes;
    type = s.type; _single_element_size = s._single_element_size;
    data = s.data; _shared = s._shared; _pinned = s._pinned; _init = s._init;
    if (_shared != nullptr) ++(*_shared);
    return *this;
}

void decx::_Vector::Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) {
    const int ns = decx::element_size(_new_type);
    if (ns == 0 || !_init) return;
    const uint64_t bytes = length * uint64_t(_single_element_size);
    if (bytes % uint64_t(ns) != 0) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
        return;
    }
    type = _new_type;
    _single_element_size = ns;
    length = bytes / uint64_t(ns);
    _length = total_bytes / uint64_t(ns);
}

decx::_Vector::~_Vector() { release(); }

// ------------------------------------------------------------------------------------------------ device vector
decx::_GPU_Vector::_GPU_Vector() {}
decx::_GPU_Vector::_GPU_Vector(const de::_DATA_TYPES_FLAGS_ t, uint64_t len) { construct(t, len); }

void decx::_GPU_Vector::construct(const de::_DATA_TYPES_FLAGS_ t, uint64_t len) {
    release();
    type = t;
    _single_element_size = decx::element_size(t);
    length = len;
    _length = padded(len, 4);
    total_bytes = _length * uint64_t(_single_element_size);
    if (total_bytes == 0) return;
    cudaGetDevice(&_device);
    if (decx::alloc::_device_malloc(&Vec, total_bytes, true, nullptr) != 0) {
        cudaGetLastError();
        decx::err::set(de::GetLastError(), de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
        total_bytes = 0;
        return;
    }
    _init = true;
}

void decx::_GPU_Vector::re_construct(const de::_DATA_TYPES_FLAGS_ t, uint64_t len) {
    int now_dev = 0;
    cudaGetDevice(&now_dev);
    const bool usable = Vec.block != nullptr && !Vec.block->orphan &&
                        Vec.block->pool == decx::MemPool_D::GetInstance(now_dev);
    if (_init && usable && t == type && len == length) return;
    const uint64_t need = padded(len, 4) * uint64_t(decx::element_size(t));
    if (_init && usable && Vec.block->size >= need && Vec.block->refcount == 1) {
        type = t;
        _single_element_size = decx::element_size(t);
        length = len;
        _length = padded(len, 4);
        total_bytes = need;
        return;
    }
    construct(t, len);
}

size_t decx::_GPU_Vector::Len() const { return length; }
de::_DATA_TYPES_FLAGS_ decx::_GPU_Vector::Type() const { return type; }

void decx::_GPU_Vector::release() {
    if (Vec.block != nullptr) decx::alloc::_device_dealloc(&Vec);     // the block knows its pool
    _init = false;
    total_bytes = 0;
    length = _length = 0;
}

de::GPU_Vector& decx::_GPU_Vector::SoftCopy(de::GPU_Vector& src) {
    decx::_GPU_Vector& s = dynamic_cast<decx::_GPU_Vector&>(src);
    if (&s == this) return *this;
    release();
    length = s.length; _length = s._length; total_bytes = s.total_bytes;
    type = s.type; _single_element_size = s._single_element_size; _device = s._device;
    Vec = s.Vec;
    if (Vec.block != nullptr) decx::alloc::_device_malloc_same_place(&Vec);
    _init = s._init;
    return *this;
}

void decx::_GPU_Vector::Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) {
    const int ns = decx::element_size(_new_type);
    if (ns == 0 || !_init) return;
    const uint64_t bytes = length * uint64_t(_single_element_size);
    if (bytes % uint64_t(ns) != 0) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
        return;
    }
    type = _new_type;
    _single_element_size = ns;
    length = bytes / uint64_t(ns);
    _length = total_bytes / uint64_t(ns);
}

decx::_GPU_Vector::~_GPU_Vector() {}      // like the device matrix: release() is the caller's call

// ------------------------------------------------------------------------------------------------ factories
de::Vector& de::CreateVectorRef() { return *(new decx::_Vector()); }
de::Vector* de::CreateVectorPtr() { return new decx::_Vector(); }
de::Vector& de::CreateVectorRef(const de::_DATA_TYPES_FLAGS_ _type, size_t len) { return *(new decx::_Vector(_type, len)); }
de::Vector* de::CreateVectorPtr(const de::_DATA_TYPES_FLAGS_ _type, size_t len) { return new decx::_Vector(_type, len); }
de::GPU_Vector& de::CreateGPUVectorRef() { return *(new decx::_GPU_Vector()); }
de::GPU_Vector* de::CreateGPUVectorPtr() { return new decx::_GPU_Vector(); }
de::GPU_Vector& de::CreateGPUVectorRef(const de::_DATA_TYPES_FLAGS_ _type, const size_t _length) {
    return *(new decx::_GPU_Vector(_type, _length));
}
de::GPU_Vector* de::CreateGPUVectorPtr(const de::_DATA_TYPES_FLAGS_ _type, const size_t _length) {
    return new decx::_GPU_Vector(_type, _length);
}

// ------------------------------------------------------------------------------------------------ pinning
de::DH de::cuda::PinMemory(de::Vector& src) {
    de::DH h;
    decx::err::success(&h);
    decx::_Vector* v = dynamic_cast<decx::_Vector*>(&src);
    if (v == nullptr || !v->_init) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (v->_pinned) {
        decx::err::set(&h, de::DECX_FAIL_HOST_MEM_REGISTERED, "error: The host memory has been registered");
    } else if (cudaHostRegister(v->data, v->total_bytes, cudaHostRegisterPortable) != cudaSuccess) {
        cudaGetLastError();
        decx::err::set(&h, de::DECX_FAIL_ALLOCATION, "error: Fail to page-lock the host memory");
    } else {
        v->_pinned = true;
    }
    return h;
}

de::DH de::cuda::UnpinMemory(de::Vector& src) {
    de::DH h;
    decx::err::success(&h);
    decx::_Vector* v = dynamic_cast<decx::_Vector*>(&src);
    if (v == nullptr || !v->_init) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (!v->_pinned) {
        decx::err::set(&h, de::DECX_FAIL_HOST_MEM_UNREGISTERED, "error: The host memory is not registered");
    } else {
        cudaHostUnregister(v->data);
        v->_pinned = false;
    }
    return h;
}

// ------------------------------------------------------------------------------------------------ de::Memcpy
de::DH de::Memcpy(de::Vector& __host, de::GPU_Vector& __device, const uint64_t start_src, const uint64_t start_dst,
                  const uint64_t cpy_size, const int _memcpy_flag) {
    de::DH h;
    decx::err::success(&h);
    decx::_Vector* hv = dynamic_cast<decx::_Vector*>(&__host);
    decx::_GPU_Vector* dv = dynamic_cast<decx::_GPU_Vector*>(&__device);
    if (!decx::cuda::_is_CUDA_init()) {
        decx::err::set(&h, de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first");
    } else if (hv == nullptr || dv == nullptr || !hv->_init || !dv->_init) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (hv->type != dv->type) {
        decx::err::set(&h, de::DECX_FAIL_TYPE_MOT_MATCH, "error: The types of the two objects are not equal");
    } else if (_memcpy_flag != de::DECX_MEMCPY_H2D && _memcpy_flag != de::DECX_MEMCPY_D2H) {
        decx::err::set(&h, de::DECX_FAIL_ErrorFlag, "error: This flag is meaningless in current context");
    } else {
        const bool h2d = _memcpy_flag == de::DECX_MEMCPY_H2D;
        const uint64_t slen = h2d ? hv->length : dv->length, dlen = h2d ? dv->length : hv->length;
        const uint64_t es = uint64_t(hv->_single_element_size);
        if (start_src + cpy_size > slen || start_dst + cpy_size > dlen) {
            decx::err::set(&h, de::DECX_FAIL_MEMCPY_OVERRANGED, "error: The copy area exceeds the vector");
        } else if (cpy_size > 0) {
            uint8_t* hp = static_cast<uint8_t*>(hv->data);
            uint8_t* dp = static_cast<uint8_t*>(dv->Vec.ptr);
            const cudaError_t e = h2d ? cudaMemcpy(dp + start_dst * es, hp + start_src * es, cpy_size * es, cudaMemcpyHostToDevice)
                                      : cudaMemcpy(hp + start_dst * es, dp + start_src * es, cpy_size * es, cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) {
                cudaGetLastError();
                decx::err::set(&h, de::DECX_FAIL_CUDA_STREAM, cudaGetErrorString(e));
            }
        }
    }
    if (h.error_type != de::DECX_SUCCESS) decx::err::set(de::GetLastError(), h.error_type, h.error_string);
    return h;
}
