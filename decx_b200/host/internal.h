// Internal declarations of the host layer (namespace decx), the counterpart of the reference's
// srcs/modules/core/** and srcs/common/Classes/** for the dense-GEMM path: concrete containers, the pooled
// device allocator, stream / event pools, the resource manager and the error helpers.  Names and call
// semantics follow the reference so that its other modules could link against these services; the
// implementations are new.  Everything is per device where the reference assumed one GPU.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <ctime>
#include <mutex>
#include <vector>

#include "../../include/DECX.h"

namespace decx {

// ------------------------------------------------------------------------------------------------ errors
namespace err {
// Writes code and message into `handle` (reference: decx::err::handle_error_info_modify,
// srcs/common/Handle/decx_handle.h:200-260).  Never prints, never exits.
_DECX_API_ void set(de::DH* handle, int code, const char* message);
_DECX_API_ void success(de::DH* handle);
}  // namespace err

// ------------------------------------------------------------------------------------------------ streams, events
// Pooled wrappers (reference: srcs/modules/core/cudaStream_management/cudaStream_package.h:45-79,
// cudaEvent_package.h:46-80).  get_* returns an idle object created with the requested flag on the current
// device, or makes one; detach() hands it back.
class _DECX_API_ cuda_stream {
public:
    cudaStream_t _S = nullptr;
    unsigned _flag = 0;
    int _device = 0;
    bool _is_occupied = false;

    void attach() { _is_occupied = true; }
    void detach() { _is_occupied = false; }
    void synchronize();
    cudaStream_t& get_raw_stream_ref() { return _S; }
    cudaStream_t* get_raw_stream_ptr() { return &_S; }
    void release();
};

class _DECX_API_ cuda_event {
public:
    cudaEvent_t _E = nullptr;
    unsigned _flag = 0;
    int _device = 0;
    bool _is_occupied = false;

    void attach() { _is_occupied = true; }
    void detach() { _is_occupied = false; }
    void synchronize();
    void event_record(decx::cuda_stream* attached_stream);
    cudaEvent_t& get_raw_event_ref() { return _E; }
    cudaEvent_t* get_raw_event_ptr() { return &_E; }
    void release();
};

namespace cuda {
_DECX_API_ decx::cuda_stream* get_cuda_stream_ptr(const int flag);   // nullptr on failure
_DECX_API_ decx::cuda_event* get_cuda_event_ptr(const int flag);
// reference forms of the two calls above (cudaStream_package.h:81-90, cudaEvent_package.h): the caller must
// know that a stream / event can be had -- on failure these return a static, never-attached dummy whose raw
// handle is null
_DECX_API_ decx::cuda_stream& get_cuda_stream_ref(const int flag);
_DECX_API_ decx::cuda_event& get_cuda_event_ref(const int flag);
_DECX_API_ void release_stream_event_pools();
_DECX_API_ size_t pooled_stream_count();
_DECX_API_ size_t pooled_event_count();
// test hook: replace stream / event creation and destruction and the "current device" query (nullptr = CUDA)
struct RawHooks {
    int (*stream_create)(cudaStream_t*, unsigned);
    int (*stream_destroy)(cudaStream_t);
    int (*event_create)(cudaEvent_t*, unsigned);
    int (*event_destroy)(cudaEvent_t);
    int (*current_device)();
};
_DECX_API_ void set_raw_hooks(const RawHooks* hooks);
_DECX_API_ bool _is_CUDA_init();
_DECX_API_ const cudaDeviceProp& _get_cuda_prop();
}  // namespace cuda

// ------------------------------------------------------------------------------------------------ device pool
class MemPool_D;
// One block of a pooled chunk (reference: srcs/modules/core/memory_management/MemBlock.h:46-96).
struct MemBlock {
    MemPool_D* pool = nullptr;  // the pool (= device) the block belongs to: it is always returned there
    uint8_t* ptr = nullptr;
    uint64_t size = 0;          // bytes, a multiple of 256
    bool idle = true;
    int refcount = 0;
    int chunk = -1;             // index of the owning chunk
    bool orphan = false;        // the pool was released while references were alive: memory gone, metadata kept
    MemBlock* prev = nullptr;   // neighbours inside the chunk, in address order
    MemBlock* next = nullptr;
};

template <typename T>
struct PtrInfo {
    decx::MemBlock* block = nullptr;
    T* ptr = nullptr;
};

// Pooled device allocator (reference: MemPool_D / MemChunk_D, srcs/modules/core/memory_management/
// MemoryPool_D.cu:47-151, MemChunk_D.cu:58-232): physical chunks of 2^k bytes (k >= 20 here) come from
// the raw allocator, requests are carved first-fit out of idle blocks, freed blocks merge with idle
// neighbours, nothing goes back to CUDA before release().  Differences from the reference, on purpose:
// one pool per device; every block starts on a 256-byte boundary (the reference carves at raw request
// sizes, which breaks TMA's 16-byte rule); blocks are reference counted so SoftCopy can share them.
class _DECX_API_ MemPool_D {
public:
    typedef int (*raw_alloc_fn)(void** p, size_t bytes);
    typedef int (*raw_free_fn)(void* p);

    static MemPool_D* GetInstance(int device);
    // test hook: replace cudaMalloc / cudaFree (for every pool created afterwards and the existing ones)
    static void set_raw_allocator(raw_alloc_fn a, raw_free_fn f);

    int allocate(uint64_t bytes, decx::MemBlock** out);   // 0 or a cudaError_t value
    void register_reference(decx::MemBlock* b);
    void deallocate(decx::MemBlock* b);                   // drops one reference; frees at zero
    void release();                                       // returns every chunk to the raw allocator

    // introspection for tests
    uint64_t bytes_reserved() const;
    uint64_t bytes_in_use() const;
    size_t chunk_count() const;
    size_t idle_block_count() const;
    bool check_invariants() const;

private:
    struct Chunk { uint8_t* base; uint64_t size; MemBlock* first; };
    mutable std::mutex _mtx;
    std::vector<Chunk> _chunks;
    void merge_with_next(MemBlock* b);
};

namespace alloc {
// (reference: decx::alloc::_device_malloc/_device_realloc/_device_dealloc/_device_malloc_same_place,
// srcs/modules/core/allocators.h:61-238).  Pool of the CURRENT device.  Return 0 on success.
_DECX_API_ int _device_malloc(decx::PtrInfo<void>* p, uint64_t bytes, bool set_zero = false, decx::cuda_stream* S = nullptr);
_DECX_API_ int _device_realloc(decx::PtrInfo<void>* p, uint64_t bytes, bool set_zero = false, decx::cuda_stream* S = nullptr);
_DECX_API_ void _device_dealloc(decx::PtrInfo<void>* p);
_DECX_API_ void _device_malloc_same_place(decx::PtrInfo<void>* p);   // share: one more reference to p->block

// Block-level interface other DECX modules link against (reference: srcs/modules/core/decx_alloc_interface.h:45-96).
// Pool of the current device; 0 on success, -1 on failure.
_DECX_API_ int _alloc_D(decx::MemBlock** _ptr, size_t req_size);
_DECX_API_ void _alloc_D_same_place(decx::MemBlock** _ptr);
_DECX_API_ void _dealloc_D(decx::MemBlock* _ptr);
_DECX_API_ void Memset_D(decx::MemBlock* _ptr, const size_t size, const int value, cudaStream_t* S);
}  // namespace alloc

// Generic cached resources with a lifespan (reference: decx::ResourceCheckIn/Lock/Unlock/CheckOut,
// srcs/modules/core/resources_manager/decx_resource.h:67-76, ResMgr.cxx:86-125).  *exposed_ptr is an object the
// caller built; once it has been unlocked and idle for lifespan_sec the collector thread calls _decon(*exposed_ptr)
// -- which must free it -- and sets *exposed_ptr to NULL, so the caller rebuilds it on next use.  Lock / Unlock
// are "in use" marks for the collector (Unlock restarts the idle clock), not mutual exclusion between users.
typedef void (*res_release_fn)(void*);
_DECX_API_ uint64_t ResourceCheckIn(void** exposed_ptr, const time_t lifespan_sec, res_release_fn _decon);
_DECX_API_ void ResourceLock(const uint64_t res_id);
_DECX_API_ void ResourceUnlock(const uint64_t res_id);
_DECX_API_ void ResourceCheckOut(const uint64_t res_id);
namespace alloc {}

// ------------------------------------------------------------------------------------------------ resources
// Cache of rebuildable scratch with a lifespan (reference: decx::ResourceHandle / decx::ResMgr,
// srcs/modules/core/resources_manager/decx_resource.h:173-225, ResMgr.cxx:47-132: GEMM planners register
// with 5 s).  Here the cached resource is the GEMM workspace / staging arena of a device; a background
// thread returns it to the pool once it has been idle for its lifespan.  lock()/unlock() are real mutual
// exclusion here (in the reference they are only "in use" marks for the collector).
class _DECX_API_ ScratchResource {
public:
    explicit ScratchResource(double lifespan_seconds = 5.0);
    ~ScratchResource();
    // Locks the resource and returns at least `bytes` of device scratch of the current device (grow-only
    // while in use); nullptr on allocation failure (lock released).  Pair with unlock().
    void* lock(uint64_t bytes, int device);
    void unlock();
    void collect_if_idle(double now);      // called by the manager thread
    void release_now();
    uint64_t capacity() const { return _bytes; }

private:
    std::mutex _mtx;
    decx::PtrInfo<void> _mem;
    uint64_t _bytes = 0;
    int _device = -1;
    double _lifespan, _last_used = 0.0;
};

namespace res {
_DECX_API_ void register_resource(decx::ScratchResource* r);
_DECX_API_ void unregister_resource(decx::ScratchResource* r);
_DECX_API_ void release_all();
_DECX_API_ double now_seconds();
}  // namespace res

// ------------------------------------------------------------------------------------------------ containers
// (reference: decx::_matrix_layout, decx::_Matrix, decx::_GPU_Matrix -- srcs/common/Classes/Matrix.h:91-267,
// GPU_Matrix.h:105-188, srcs/modules/core/classes/Matrix.cxx, GPU_Matrix.cu)
inline int element_size(de::_DATA_TYPES_FLAGS_ t) {
    switch (t) {
        case de::_FP16_: return 2;
        case de::_FP32_: case de::_INT32_: case de::_UCHAR4_: return 4;
        case de::_FP64_: case de::_COMPLEX_F32_: case de::_UINT64_: return 8;
        case de::_COMPLEX_F64_: case de::_VECTOR4F_: case de::_VECTOR3F_: return 16;
        case de::_UINT8_: return 1;
        default: return 0;
    }
}
// pitch in elements: width rounded up to `align_bytes` bytes (32 on the host, 128 on the device)
inline uint32_t pitch_for(uint32_t width, int esize, uint32_t align_bytes) {
    if (esize <= 0) return width;
    const uint64_t bytes = (uint64_t(width) * esize + align_bytes - 1) / align_bytes * align_bytes;
    return uint32_t(bytes / esize);
}

class _DECX_API_ _Matrix : public de::Matrix {
public:
    de::MatrixLayout _layout;
    de::_DATA_TYPES_FLAGS_ type = de::_VOID_;
    de::_DATA_FORMATS_ _format = de::_NA_;
    bool _init = false, _pinned = false, _owner = false;
    uint64_t total_bytes = 0;
    void* data = nullptr;          // 64-byte aligned, zero-filled
    int* _shared = nullptr;        // reference count shared by soft copies

    _Matrix();
    _Matrix(const de::_DATA_TYPES_FLAGS_ type, const uint32_t width, const uint32_t height,
            const de::_DATA_FORMATS_ format = de::_NA_);
    void construct(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height,
                   const de::_DATA_FORMATS_ format = de::_NA_);
    void re_construct(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height);

    virtual uint32_t Width() const;
    virtual uint32_t Height() const;
    virtual void release();
    virtual de::Matrix& SoftCopy(de::Matrix& src);
    virtual de::_DATA_TYPES_FLAGS_ Type() const;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type);
    virtual de::_DATA_FORMATS_ Format() const;
    virtual ~_Matrix();
    uint32_t Pitch() const { return _layout.pitch; }
};

class _DECX_API_ _GPU_Matrix : public de::GPU_Matrix {
public:
    de::MatrixLayout _layout;
    de::_DATA_TYPES_FLAGS_ type = de::_VOID_;
    de::_DATA_FORMATS_ _format = de::_NA_;
    bool _init = false;
    uint64_t total_bytes = 0;
    int _device = -1;                 // ordinal the storage lives on (the reference is single-GPU)
    decx::PtrInfo<void> Mat;

    _GPU_Matrix();
    _GPU_Matrix(const de::_DATA_TYPES_FLAGS_ type, const uint32_t width, const uint32_t height,
                const de::_DATA_FORMATS_ format = de::_NA_);
    void construct(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height,
                   const de::_DATA_FORMATS_ format = de::_NA_);
    // new shape; re-allocates only if more bytes are needed (reference: GPU_Matrix.cu:120-134)
    void re_construct(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, decx::cuda_stream* S = nullptr);

    virtual uint Width() const;
    virtual uint Height() const;
    virtual void release();
    virtual de::_DATA_TYPES_FLAGS_ Type() const;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type);
    virtual de::GPU_Matrix& SoftCopy(de::GPU_Matrix& src);
    virtual de::_DATA_FORMATS_ Format() const;
    virtual ~_GPU_Matrix();
    uint32_t Pitch() const { return _layout.pitch; }
};

// ------------------------------------------------------------------------------------------------ vectors
// (reference: decx::_Vector srcs/common/Classes/Vector.h:118-180, decx::_GPU_Vector GPU_Vector.h:77-140)
class _DECX_API_ _Vector : public de::Vector {
public:
    uint64_t length = 0, _length = 0, total_bytes = 0;      // logical, padded to 8 elements, bytes of the padding
    de::_DATA_TYPES_FLAGS_ type = de::_VOID_;
    int _single_element_size = 0;
    bool _init = false, _pinned = false;
    void* data = nullptr;           // 64-byte aligned, zero-filled
    int* _shared = nullptr;

    _Vector();
    _Vector(const de::_DATA_TYPES_FLAGS_ type, uint64_t length);
    void construct(const de::_DATA_TYPES_FLAGS_ type, uint64_t length);
    void re_construct(const de::_DATA_TYPES_FLAGS_ type, uint64_t length);

    virtual size_t Len() const;
    virtual void release();
    virtual de::Vector& SoftCopy(de::Vector& src);
    virtual de::_DATA_TYPES_FLAGS_ Type() const;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type);
    virtual ~_Vector();
};

class _DECX_API_ _GPU_Vector : public de::GPU_Vector {
public:
    uint64_t length = 0, _length = 0, total_bytes = 0;      // padded to 4 elements
    de::_DATA_TYPES_FLAGS_ type = de::_VOID_;
    int _single_element_size = 0;
    bool _init = false;
    int _device = -1;
    decx::PtrInfo<void> Vec;

    _GPU_Vector();
    _GPU_Vector(const de::_DATA_TYPES_FLAGS_ type, uint64_t length);
    void construct(const de::_DATA_TYPES_FLAGS_ type, uint64_t length);
    void re_construct(const de::_DATA_TYPES_FLAGS_ type, uint64_t length);

    virtual size_t Len() const;
    virtual void release();
    virtual de::GPU_Vector& SoftCopy(de::GPU_Vector& src);
    virtual de::_DATA_TYPES_FLAGS_ Type() const;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type);
    virtual ~_GPU_Vector();
};

// ------------------------------------------------------------------------------------------------ tensors
// (reference: decx::_Tensor srcs/common/Classes/Tensor.h:59-82 + srcs/modules/core/classes/Tensor.cxx,
// decx::_TensorArray TensorArray.cxx, decx::_GPU_Tensor GPU_Tensor.cu:35-140, decx::_GPU_TensorArray
// srcs/common/Classes/GPU_TensorArray.h:115-200).  Channels innermost; see include/DECX/classes/tensors.h.
_DECX_API_ void tensor_layout(de::TensorLayout& l, de::_DATA_TYPES_FLAGS_ t, uint32_t width, uint32_t height,
                              uint32_t depth, uint32_t width_align);

class _DECX_API_ _Tensor : public de::Tensor {
public:
    de::TensorLayout _layout;
    de::_DATA_TYPES_FLAGS_ type = de::_VOID_;
    bool _init = false, _pinned = false, _view = false;    // _view: a slice of a tensor array
    uint64_t total_bytes = 0;
    void* data = nullptr;            // 64-byte aligned, zero-filled
    void* base = nullptr;            // start of the allocation `data` lies in (differs for a slice)
    int* _shared = nullptr;          // owners of the allocation: tensors, slices and the array itself

    _Tensor();
    _Tensor(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, uint32_t depth);
    void construct(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, uint32_t depth);

    virtual uint32_t Width() const;
    virtual uint32_t Height() const;
    virtual uint32_t Depth() const;
    virtual de::Tensor& SoftCopy(de::Tensor& src);
    virtual void release();
    virtual de::_DATA_TYPES_FLAGS_ Type() const;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type);
    virtual ~_Tensor();
};

class _DECX_API_ _TensorArray : public de::TensorArray {
public:
    de::TensorLayout _layout;
    de::_DATA_TYPES_FLAGS_ type = de::_VOID_;
    uint32_t tensor_num = 0;
    bool _init = false;
    uint64_t _gap = 0, total_bytes = 0;     // elements between two tensors; bytes of all of them
    void* data = nullptr;
    void** ptrs = nullptr;                  // base pointer of every tensor (what ptr<T>() indexes)
    int* _shared = nullptr;

    _TensorArray();
    _TensorArray(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, uint32_t depth, uint32_t tensor_num);
    void construct(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, uint32_t depth, uint32_t tensor_num);

    virtual uint32_t Width() const;
    virtual uint32_t Height() const;
    virtual uint32_t Depth() const;
    virtual uint32_t TensorNum() const;
    virtual de::TensorArray& SoftCopy(de::TensorArray& src);
    virtual de::_DATA_TYPES_FLAGS_ Type() const;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type);
    virtual de::DH Extract_SoftCopy(const uint32_t index, de::Tensor& dst) const;
    virtual void release();
    virtual ~_TensorArray();
};

class _DECX_API_ _GPU_Tensor : public de::GPU_Tensor {
public:
    de::TensorLayout _layout;
    de::_DATA_TYPES_FLAGS_ type = de::_VOID_;
    bool _init = false;
    uint64_t total_bytes = 0;
    int _device = -1;
    decx::PtrInfo<void> Tens;        // a slice of a tensor array shares the array's block (reference count)

    _GPU_Tensor();
    _GPU_Tensor(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, uint32_t depth);
    void construct(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, uint32_t depth);
    // new shape; re-allocates only if more bytes are needed (reference: GPU_Tensor.cu re_construct)
    void re_construct(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, uint32_t depth,
                      decx::cuda_stream* S = nullptr);

    virtual uint32_t Width() const;
    virtual uint32_t Height() const;
    virtual uint32_t Depth() const;
    virtual de::GPU_Tensor& SoftCopy(de::GPU_Tensor& src);
    virtual void release();
    virtual de::_DATA_TYPES_FLAGS_ Type() const;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type);
    virtual de::DH Extract_SoftCopy(const uint32_t index, de::GPU_Tensor& dst) const;
    virtual ~_GPU_Tensor();
};

class _DECX_API_ _GPU_TensorArray : public de::GPU_TensorArray {
public:
    de::TensorLayout _layout;
    de::_DATA_TYPES_FLAGS_ type = de::_VOID_;
    uint32_t tensor_num = 0;
    bool _init = false;
    uint64_t _gap = 0, total_bytes = 0;     // elements between two tensors; bytes of all of them
    int _device = -1;
    decx::PtrInfo<void> TensArr;

    _GPU_TensorArray();
    _GPU_TensorArray(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, uint32_t depth, uint32_t tensor_num);
    void construct(const de::_DATA_TYPES_FLAGS_ type, uint32_t width, uint32_t height, uint32_t depth, uint32_t tensor_num);

    virtual uint32_t Width() const;
    virtual uint32_t Height() const;
    virtual uint32_t Depth() const;
    virtual uint32_t TensorNum() const;
    virtual de::_DATA_TYPES_FLAGS_ Type() const;
    virtual void Reinterpret(const de::_DATA_TYPES_FLAGS_ _new_type);
    virtual de::GPU_TensorArray& SoftCopy(const de::GPU_TensorArray& src);
    virtual de::DH Extract_SoftCopy(const uint32_t index, de::GPU_Tensor& dst) const;
    virtual void release();
    virtual ~_GPU_TensorArray();
};

}  // namespace decx
