// de::Tensor / de::TensorArray / de::GPU_Tensor / de::GPU_TensorArray objects, their factories, pinning and de::Memcpy
// (reference: srcs/modules/core/classes/Tensor.cxx, TensorArray.cxx, GPU_Tensor.cu, GPU_TensorArray.cu;
// srcs/modules/core/data transmission/data_transmission.cu:183-300).  Fresh implementations behind the reference's
// interfaces: the operands of de::nn::cuda::Conv2D.
#include <cstdlib>
#include <cstring>

#include "internal.h"

namespace {
uint64_t round_to(uint64_t n, uint64_t to) { return (n + to - 1) / to * to; }

struct DeviceGuard {            // device memory goes back to the pool of the device it came from
    int cur = 0, want;
    explicit DeviceGuard(int device) : want(device) {
        cudaGetDevice(&cur);
        if (want >= 0 && want != cur) cudaSetDevice(want);
    }
    ~DeviceGuard() {
        if (want >= 0 && want != cur) cudaSetDevice(cur);
    }
};
}  // namespace

// dpitch: depth rounded up to 16 bytes of elements (reference: _TENSOR_ALIGN_DEPTH_*, Tensor.h:40-44);
// wpitch: width rounded up to `width_align` columns (4 on the host, Tensor.cxx:44; 8 on the device, GPU_Tensor.cu:45,79)
void decx::tensor_layout(de::TensorLayout& l, de::_DATA_TYPES_FLAGS_ t, uint32_t width, uint32_t height, uint32_t depth,
                         uint32_t width_align) {
    const int es = decx::element_size(t);
    l.width = width;
    l.height = height;
    l.depth = depth;
    l._single_element_size = uint8_t(es);
    const uint32_t dalign = es > 0 && es <= 16 ? uint32_t(16 / es) : 1u;
    l.dpitch = uint32_t(round_to(depth, dalign));
    l.wpitch = uint32_t(round_to(width, width_align));
    l.dp_x_wp = uint64_t(l.dpitch) * l.wpitch;
    l.plane[0] = uint64_t(height) * width;
    l.plane[1] = uint64_t(depth) * width;
    l.plane[2] = uint64_t(height) * depth;
}

// ------------------------------------------------------------------------------------------------ host tensor
decx::_Tensor::_Tensor() {
    std::memset(&_layout, 0, sizeof(_layout));
    _exp_data_ptr = &data;
    _exp_tensor_dscr = &_layout;
}
decx::_Tensor::_Tensor(const de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t d) : _Tensor() { construct(t, w, h, d); }

void decx::_Tensor::construct(const de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t d) {
    release();
    type = t;
    decx::tensor_layout(_layout, t, w, h, d, 4);
    total_bytes = _layout.dp_x_wp * h * _layout._single_element_size;
    if (total_bytes == 0) return;
    data = std::aligned_alloc(64, round_to(total_bytes, 64));
    if (data == nullptr) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_ALLOCATION, "error: Fail to allocate memory on RAM");
        total_bytes = 0;
        return;
    }
    std::memset(data, 0, round_to(total_bytes, 64));
    base = data;
    _shared = new int(1);
    _init = true;
}

uint32_t decx::_Tensor::Width() const { return _layout.width; }
uint32_t decx::_Tensor::Height() const { return _layout.height; }
uint32_t decx::_Tensor::Depth() const { return _layout.depth; }
de::_DATA_TYPES_FLAGS_ decx::_Tensor::Type() const { return type; }

void decx::_Tensor::release() {
    if (_shared != nullptr && --(*_shared) == 0) {          // the last owner (tensor, slice or array) frees the storage
        if (_pinned) cudaHostUnregister(base);
        std::free(base);
        delete _shared;
    }
    _shared = nullptr;
    data = base = nullptr;
    _init = _pinned = _view = false;
    total_bytes = 0;
}

de::Tensor& decx::_Tensor::SoftCopy(de::Tensor& src) {
    decx::_Tensor& s = dynamic_cast<decx::_Tensor&>(src);
    if (&s == this) return *this;
    release();
    _layout = s._layout;
    type = s.type;
    total_bytes = s.total_bytes;
    data = s.data;
    base = s.base;
    _shared = s._shared;
    _pinned = s._pinned;
    _view = s._view;
    _init = s._init;
    if (_shared != nullptr) ++(*_shared);
    return *this;
}

void decx::_Tensor::Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) {
    const int ns = decx::element_size(_new_type);
    if (!_init || ns == 0) return;
    const uint64_t dbytes = uint64_t(_layout.dpitch) * _layout._single_element_size;
    if ((uint64_t(_layout.depth) * _layout._single_element_size) % uint64_t(ns) != 0 || dbytes % uint64_t(ns) != 0) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
        return;
    }
    _layout.depth = uint32_t(uint64_t(_layout.depth) * _layout._single_element_size / uint64_t(ns));
    _layout.dpitch = uint32_t(dbytes / uint64_t(ns));
    _layout.dp_x_wp = uint64_t(_layout.dpitch) * _layout.wpitch;
    _layout._single_element_size = uint8_t(ns);
    _layout.plane[1] = uint64_t(_layout.depth) * _layout.width;
    _layout.plane[2] = uint64_t(_layout.height) * _layout.depth;
    type = _new_type;
}

decx::_Tensor::~_Tensor() { release(); }

// ------------------------------------------------------------------------------------------------ host tensor array
decx::_TensorArray::_TensorArray() {
    std::memset(&_layout, 0, sizeof(_layout));
    _exp_data_ptr = &ptrs;
    _exp_tensor_dscr = &_layout;
}
decx::_TensorArray::_TensorArray(const de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t d, uint32_t n)
    : _TensorArray() {
    construct(t, w, h, d, n);
}

void decx::_TensorArray::construct(const de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t d, uint32_t n) {
    release();
    type = t;
    tensor_num = n;
    decx::tensor_layout(_layout, t, w, h, d, 4);
    _gap = _layout.dp_x_wp * h;
    total_bytes = _gap * n * _layout._single_element_size;
    if (total_bytes == 0) return;
    data = std::aligned_alloc(64, round_to(total_bytes, 64));
    ptrs = static_cast<void**>(std::malloc(sizeof(void*) * n));
    if (data == nullptr || ptrs == nullptr) {
        std::free(data);
        std::free(ptrs);
        data = nullptr;
        ptrs = nullptr;
        decx::err::set(de::GetLastError(), de::DECX_FAIL_ALLOCATION, "error: Fail to allocate memory on RAM");
        total_bytes = 0;
        return;
    }
    std::memset(data, 0, round_to(total_bytes, 64));
    for (uint32_t i = 0; i < n; ++i) ptrs[i] = static_cast<uint8_t*>(data) + uint64_t(i) * _gap * _layout._single_element_size;
    _shared = new int(1);
    _init = true;
}

uint32_t decx::_TensorArray::Width() const { return _layout.width; }
uint32_t decx::_TensorArray::Height() const { return _layout.height; }
uint32_t decx::_TensorArray::Depth() const { return _layout.depth; }
uint32_t decx::_TensorArray::TensorNum() const { return tensor_num; }
de::_DATA_TYPES_FLAGS_ decx::_TensorArray::Type() const { return type; }

void decx::_TensorArray::release() {
    if (_shared != nullptr && --(*_shared) == 0) {
        std::free(data);
        delete _shared;
    }
    std::free(ptrs);                        // every array object has its own pointer table
    ptrs = nullptr;
    _shared = nullptr;
    data = nullptr;
    _init = false;
    total_bytes = 0;
    tensor_num = 0;
}

de::TensorArray& decx::_TensorArray::SoftCopy(de::TensorArray& src) {
    decx::_TensorArray& s = dynamic_cast<decx::_TensorArray&>(src);
    if (&s == this) return *this;
    release();
    _layout = s._layout;
    type = s.type;
    tensor_num = s.tensor_num;
    _gap = s._gap;
    total_bytes = s.total_bytes;
    data = s.data;
    _shared = s._shared;
    _init = s._init;
    if (s.ptrs != nullptr) {
        ptrs = static_cast<void**>(std::malloc(sizeof(void*) * tensor_num));
        if (ptrs != nullptr) std::memcpy(ptrs, s.ptrs, sizeof(void*) * tensor_num);
    }
    if (_shared != nullptr) ++(*_shared);
    return *this;
}

void decx::_TensorArray::Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) {
    const int ns = decx::element_size(_new_type);
    if (!_init || ns == 0) return;
    if (ns != int(_layout._single_element_size)) {          // the shape stays: same element size only
        decx::err::set(de::GetLastError(), de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
        return;
    }
    type = _new_type;
}

// dst becomes a view of tensor `index`: same storage, no copy (reference: TensorArray.cxx Extract_SoftCopy)
de::DH decx::_TensorArray::Extract_SoftCopy(const uint32_t index, de::Tensor& dst) const {
    de::DH h;
    decx::err::success(&h);
    decx::_Tensor* d = dynamic_cast<decx::_Tensor*>(&dst);
    if (d == nullptr || !_init) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (index >= tensor_num) {
        decx::err::set(&h, de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
    } else {
        d->release();
        d->_layout = _layout;
        d->type = type;
        d->total_bytes = _gap * _layout._single_element_size;
        d->data = ptrs[index];
        d->base = data;
        d->_shared = _shared;
        ++(*_shared);
        d->_view = true;
        d->_init = true;
    }
    if (h.error_type != de::DECX_SUCCESS) decx::err::set(de::GetLastError(), h.error_type, h.error_string);
    return h;
}

decx::_TensorArray::~_TensorArray() { release(); }

// ------------------------------------------------------------------------------------------------ device tensor
decx::_GPU_Tensor::_GPU_Tensor() { std::memset(&_layout, 0, sizeof(_layout)); }
decx::_GPU_Tensor::_GPU_Tensor(const de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t d) : _GPU_Tensor() {
    construct(t, w, h, d);
}

void decx::_GPU_Tensor::construct(const de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t d) {
    release();
    type = t;
    decx::tensor_layout(_layout, t, w, h, d, 8);
    total_bytes = _layout.dp_x_wp * h * _layout._single_element_size;
    if (total_bytes == 0) return;
    cudaGetDevice(&_device);
    if (decx::alloc::_device_malloc(&Tens, total_bytes, true, nullptr) != 0) {
        cudaGetLastError();
        decx::err::set(de::GetLastError(), de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
        total_bytes = 0;
        return;
    }
    _init = true;
}

void decx::_GPU_Tensor::re_construct(const de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t d,
                                     decx::cuda_stream* S) {
    // a block is only kept if this object is its only owner (not a slice of an array) and it lives in the pool of
    // the device that is current now
    int now_dev = 0;
    cudaGetDevice(&now_dev);
    const bool usable = Tens.block != nullptr && !Tens.block->orphan && Tens.block->refcount == 1 &&
                        Tens.block->pool == decx::MemPool_D::GetInstance(now_dev) && Tens.ptr == Tens.block->ptr;
    if (_init && usable && t == type && w == _layout.width && h == _layout.height && d == _layout.depth) return;
    de::TensorLayout nl;
    decx::tensor_layout(nl, t, w, h, d, 8);
    const uint64_t need = nl.dp_x_wp * h * nl._single_element_size;
    if (_init && usable && Tens.block->size >= need) {
        type = t;
        _layout = nl;
        total_bytes = need;                           // grow-only: the block is kept
        return;
    }
    release();
    type = t;
    _layout = nl;
    total_bytes = need;
    if (need == 0) return;
    cudaGetDevice(&_device);
    if (decx::alloc::_device_malloc(&Tens, need, true, S) != 0) {
        cudaGetLastError();
        decx::err::set(de::GetLastError(), de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
        total_bytes = 0;
        return;
    }
    _init = true;
}

uint32_t decx::_GPU_Tensor::Width() const { return _layout.width; }
uint32_t decx::_GPU_Tensor::Height() const { return _layout.height; }
uint32_t decx::_GPU_Tensor::Depth() const { return _layout.depth; }
de::_DATA_TYPES_FLAGS_ decx::_GPU_Tensor::Type() const { return type; }

void decx::_GPU_Tensor::release() {
    if (Tens.block != nullptr) {
        DeviceGuard g(_device);
        decx::alloc::_device_dealloc(&Tens);
    }
    Tens.block = nullptr;
    Tens.ptr = nullptr;
    _init = false;
    total_bytes = 0;
}

de::GPU_Tensor& decx::_GPU_Tensor::SoftCopy(de::GPU_Tensor& src) {
    decx::_GPU_Tensor& s = dynamic_cast<decx::_GPU_Tensor&>(src);
    if (&s == this) return *this;
    release();
    _layout = s._layout;
    type = s.type;
    total_bytes = s.total_bytes;
    _device = s._device;
    Tens = s.Tens;
    if (Tens.block != nullptr) {
        DeviceGuard g(_device);
        decx::alloc::_device_malloc_same_place(&Tens);
    }
    _init = s._init;
    return *this;
}

void decx::_GPU_Tensor::Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) {
    const int ns = decx::element_size(_new_type);
    if (!_init || ns == 0) return;
    if (ns != int(_layout._single_element_size)) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
        return;
    }
    type = _new_type;
}

// A tensor holds one tensor: index 0 is the tensor itself (the slot exists in the reference's interface,
// srcs/includes/DECX/classes/GPU_Tensor.h:46)
de::DH decx::_GPU_Tensor::Extract_SoftCopy(const uint32_t index, de::GPU_Tensor& dst) const {
    de::DH h;
    decx::err::success(&h);
    if (index != 0 || !_init) {
        decx::err::set(&h, de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
        decx::err::set(de::GetLastError(), h.error_type, h.error_string);
        return h;
    }
    dst.SoftCopy(const_cast<decx::_GPU_Tensor&>(*this));
    return h;
}

decx::_GPU_Tensor::~_GPU_Tensor() { release(); }

// ------------------------------------------------------------------------------------------------ device tensor array
decx::_GPU_TensorArray::_GPU_TensorArray() { std::memset(&_layout, 0, sizeof(_layout)); }
decx::_GPU_TensorArray::_GPU_TensorArray(const de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t d, uint32_t n)
    : _GPU_TensorArray() {
    construct(t, w, h, d, n);
}

void decx::_GPU_TensorArray::construct(const de::_DATA_TYPES_FLAGS_ t, uint32_t w, uint32_t h, uint32_t d, uint32_t n) {
    release();
    type = t;
    tensor_num = n;
    decx::tensor_layout(_layout, t, w, h, d, 8);
    _gap = _layout.dp_x_wp * h;
    total_bytes = _gap * n * _layout._single_element_size;
    if (total_bytes == 0) return;
    cudaGetDevice(&_device);
    if (decx::alloc::_device_malloc(&TensArr, total_bytes, true, nullptr) != 0) {
        cudaGetLastError();
        decx::err::set(de::GetLastError(), de::DECX_FAIL_CUDA_ALLOCATION, "error: Fail to allocate memory on device");
        total_bytes = 0;
        return;
    }
    _init = true;
}

uint32_t decx::_GPU_TensorArray::Width() const { return _layout.width; }
uint32_t decx::_GPU_TensorArray::Height() const { return _layout.height; }
uint32_t decx::_GPU_TensorArray::Depth() const { return _layout.depth; }
uint32_t decx::_GPU_TensorArray::TensorNum() const { return tensor_num; }
de::_DATA_TYPES_FLAGS_ decx::_GPU_TensorArray::Type() const { return type; }

void decx::_GPU_TensorArray::release() {
    if (TensArr.block != nullptr) {
        DeviceGuard g(_device);
        decx::alloc::_device_dealloc(&TensArr);
    }
    TensArr.block = nullptr;
    TensArr.ptr = nullptr;
    _init = false;
    total_bytes = 0;
    tensor_num = 0;
}

de::GPU_TensorArray& decx::_GPU_TensorArray::SoftCopy(const de::GPU_TensorArray& src) {
    const decx::_GPU_TensorArray& s = dynamic_cast<const decx::_GPU_TensorArray&>(src);
    if (&s == this) return *this;
    release();
    _layout = s._layout;
    type = s.type;
    tensor_num = s.tensor_num;
    _gap = s._gap;
    total_bytes = s.total_bytes;
    _device = s._device;
    TensArr = s.TensArr;
    if (TensArr.block != nullptr) {
        DeviceGuard g(_device);
        decx::alloc::_device_malloc_same_place(&TensArr);
    }
    _init = s._init;
    return *this;
}

void decx::_GPU_TensorArray::Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type) {
    const int ns = decx::element_size(_new_type);
    if (!_init || ns == 0) return;
    if (ns != int(_layout._single_element_size)) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
        return;
    }
    type = _new_type;
}

// dst becomes a view of tensor `index`: it shares the array's block (one more reference), no copy
// (reference: GPU_TensorArray.cu Extract_SoftCopy)
de::DH decx::_GPU_TensorArray::Extract_SoftCopy(const uint32_t index, de::GPU_Tensor& dst) const {
    de::DH h;
    decx::err::success(&h);
    decx::_GPU_Tensor* d = dynamic_cast<decx::_GPU_Tensor*>(&dst);
    if (d == nullptr || !_init) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (index >= tensor_num) {
        decx::err::set(&h, de::DECX_FAIL_INVALID_PARAM, "error: The parameter(s) is(are) invalid");
    } else {
        d->release();
        d->_layout = _layout;
        d->type = type;
        d->total_bytes = _gap * _layout._single_element_size;
        d->_device = _device;
        d->Tens.block = TensArr.block;
        d->Tens.ptr = static_cast<uint8_t*>(TensArr.ptr) + uint64_t(index) * _gap * _layout._single_element_size;
        {
            DeviceGuard g(_device);
            decx::alloc::_device_malloc_same_place(&d->Tens);
        }
        d->_init = true;
    }
    if (h.error_type != de::DECX_SUCCESS) decx::err::set(de::GetLastError(), h.error_type, h.error_string);
    return h;
}

decx::_GPU_TensorArray::~_GPU_TensorArray() { release(); }

// ------------------------------------------------------------------------------------------------ factories, pinning
de::Tensor* de::CreateTensorPtr() { return new decx::_Tensor(); }
de::Tensor& de::CreateTensorRef() { return *new decx::_Tensor(); }
de::Tensor* de::CreateTensorPtr(const de::_DATA_TYPES_FLAGS_ t, const uint32_t w, const uint32_t h, const uint32_t d) {
    return new decx::_Tensor(t, w, h, d);
}
de::Tensor& de::CreateTensorRef(const de::_DATA_TYPES_FLAGS_ t, const uint32_t w, const uint32_t h, const uint32_t d) {
    return *new decx::_Tensor(t, w, h, d);
}
de::TensorArray& de::CreateTensorArrayRef() { return *new decx::_TensorArray(); }
de::TensorArray* de::CreateTensorArrayPtr() { return new decx::_TensorArray(); }
de::TensorArray& de::CreateTensorArrayRef(const de::_DATA_TYPES_FLAGS_ t, const uint32_t w, const uint32_t h, const uint32_t d,
                                          const uint32_t n) {
    return *new decx::_TensorArray(t, w, h, d, n);
}
de::TensorArray* de::CreateTensorArrayPtr(const de::_DATA_TYPES_FLAGS_ t, const uint32_t w, const uint32_t h, const uint32_t d,
                                          const uint32_t n) {
    return new decx::_TensorArray(t, w, h, d, n);
}
de::GPU_Tensor* de::CreateGPUTensorPtr() { return new decx::_GPU_Tensor(); }
de::GPU_Tensor& de::CreateGPUTensorRef() { return *new decx::_GPU_Tensor(); }
de::GPU_Tensor* de::CreateGPUTensorPtr(const de::_DATA_TYPES_FLAGS_ t, const uint32_t w, const uint32_t h, const uint32_t d) {
    return new decx::_GPU_Tensor(t, w, h, d);
}
de::GPU_Tensor& de::CreateGPUTensorRef(const de::_DATA_TYPES_FLAGS_ t, const uint32_t w, const uint32_t h, const uint32_t d) {
    return *new decx::_GPU_Tensor(t, w, h, d);
}
de::GPU_TensorArray& de::CreateGPUTensorArrayRef() { return *new decx::_GPU_TensorArray(); }
de::GPU_TensorArray* de::CreateGPUTensorArrayPtr() { return new decx::_GPU_TensorArray(); }
de::GPU_TensorArray& de::CreateGPUTensorArrayRef(const de::_DATA_TYPES_FLAGS_ t, const uint32_t w, const uint32_t h,
                                                 const uint32_t d, const uint32_t n) {
    return *new decx::_GPU_TensorArray(t, w, h, d, n);
}
de::GPU_TensorArray* de::CreateGPUTensorArrayPtr(const de::_DATA_TYPES_FLAGS_ t, const uint32_t w, const uint32_t h,
                                                 const uint32_t d, const uint32_t n) {
    return new decx::_GPU_TensorArray(t, w, h, d, n);
}

de::DH de::cuda::PinMemory(de::Tensor& src) {
    de::DH h;
    decx::err::success(&h);
    decx::_Tensor* m = dynamic_cast<decx::_Tensor*>(&src);
    if (m == nullptr || !m->_init || m->_view) {            // a slice is pinned (or not) with its array
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

de::DH de::cuda::UnpinMemory(de::Tensor& src) {
    de::DH h;
    decx::err::success(&h);
    decx::_Tensor* m = dynamic_cast<decx::_Tensor*>(&src);
    if (m == nullptr || !m->_init || m->_view) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (m->_pinned) {
        cudaHostUnregister(m->data);
        m->_pinned = false;
    }
    return h;
}

// ------------------------------------------------------------------------------------------------ de::Memcpy
// One 3-D copy: extent {D elements, W columns, H rows}; a stored row of columns is dpitch elements wide and a stored
// image row holds wpitch columns (the reference builds the same cudaMemcpy3DParms, data_transmission.cu:211-255).
de::DH de::Memcpy(de::Tensor& __host, de::GPU_Tensor& __device, const de::Point3D start_src, const de::Point3D start_dst,
                  const de::Point3D cpy_size, const int _memcpy_flag) {
    de::DH h;
    decx::err::success(&h);
    if (!decx::cuda::_is_CUDA_init()) {
        decx::err::set(&h, de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first");
        decx::err::set(de::GetLastError(), h.error_type, h.error_string);
        return h;
    }
    decx::_Tensor* ht = dynamic_cast<decx::_Tensor*>(&__host);
    decx::_GPU_Tensor* dt = dynamic_cast<decx::_GPU_Tensor*>(&__device);
    if (ht == nullptr || dt == nullptr || !ht->_init || !dt->_init) {
        decx::err::set(&h, de::DECX_FAIL_CLASS_NOT_INIT, "error: The class is not initialized");
    } else if (ht->type != dt->type) {
        decx::err::set(&h, de::MEMCPY_DIFFERENT_TYPES, "error: The types of the two objects are not equal");
    } else if (_memcpy_flag != de::DECX_MEMCPY_H2D && _memcpy_flag != de::DECX_MEMCPY_D2H) {
        decx::err::set(&h, de::DECX_FAIL_ErrorFlag, "error: This flag is meaningless in current context");
    } else {
        const bool h2d = (_memcpy_flag == de::DECX_MEMCPY_H2D);
        const de::TensorLayout& sl = h2d ? ht->_layout : dt->_layout;
        const de::TensorLayout& dl = h2d ? dt->_layout : ht->_layout;
        auto outside = [](const de::Point3D& s, const de::Point3D& c, const de::TensorLayout& l) {
            return s.x < 0 || s.y < 0 || s.z < 0 || c.x < 0 || c.y < 0 || c.z < 0 || uint64_t(s.x) + c.x > l.depth ||
                   uint64_t(s.y) + c.y > l.width || uint64_t(s.z) + c.z > l.height;
        };
        if (outside(start_src, cpy_size, sl) || outside(start_dst, cpy_size, dl)) {
            decx::err::set(&h, de::DECX_FAIL_MEMCPY_OVERRANGED, "error: The copy area exceeds the tensor");
        } else if (cpy_size.x > 0 && cpy_size.y > 0 && cpy_size.z > 0) {
            const uint64_t es = sl._single_element_size;
            void* sp = h2d ? ht->data : dt->Tens.ptr;
            void* dp = h2d ? dt->Tens.ptr : ht->data;
            cudaMemcpy3DParms prm;
            std::memset(&prm, 0, sizeof(prm));
            prm.srcPtr = make_cudaPitchedPtr(sp, sl.dpitch * es, sl.depth * es, sl.wpitch);
            prm.dstPtr = make_cudaPitchedPtr(dp, dl.dpitch * es, dl.depth * es, dl.wpitch);
            prm.srcPos = make_cudaPos(start_src.x * es, start_src.y, start_src.z);
            prm.dstPos = make_cudaPos(start_dst.x * es, start_dst.y, start_dst.z);
            prm.extent = make_cudaExtent(cpy_size.x * es, cpy_size.y, cpy_size.z);
            prm.kind = h2d ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost;
            const cudaError_t e = cudaMemcpy3D(&prm);
            if (e != cudaSuccess) {
                cudaGetLastError();
                decx::err::set(&h, de::DECX_FAIL_CUDA_STREAM, cudaGetErrorString(e));
            }
        }
    }
    if (h.error_type != de::DECX_SUCCESS) decx::err::set(de::GetLastError(), h.error_type, h.error_string);
    return h;
}
