// Pooled device allocator: see the class comment in internal.h.
#include <algorithm>
#include <map>

#include "internal.h"

namespace {

int cuda_raw_alloc(void** p, size_t bytes) { return int(cudaMalloc(p, bytes)); }
int cuda_raw_free(void* p) { return int(cudaFree(p)); }

decx::MemPool_D::raw_alloc_fn g_raw_alloc = cuda_raw_alloc;
decx::MemPool_D::raw_free_fn g_raw_free = cuda_raw_free;

std::mutex g_pools_mtx;
std::map<int, decx::MemPool_D*> g_pools;

constexpr uint64_t BLOCK_ALIGN = 256;          // every block starts on a 256-byte boundary
constexpr uint64_t MIN_CHUNK = 1ull << 20;     // physical chunks are powers of two, at least 1 MiB

inline uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }
inline uint64_t pow2_at_least(uint64_t x) {
    uint64_t p = MIN_CHUNK;
    while (p < x) p <<= 1;
    return p;
}

}  // namespace

decx::MemPool_D* decx::MemPool_D::GetInstance(int device) {
    std::lock_guard<std::mutex> lk(g_pools_mtx);
    auto it = g_pools.find(device);
    if (it != g_pools.end()) return it->second;
    decx::MemPool_D* p = new decx::MemPool_D;
    g_pools[device] = p;
    return p;
}

void decx::MemPool_D::set_raw_allocator(raw_alloc_fn a, raw_free_fn f) {
    g_raw_alloc = a ? a : cuda_raw_alloc;
    g_raw_free = f ? f : cuda_raw_free;
}

int decx::MemPool_D::allocate(uint64_t bytes, decx::MemBlock** out) {
    *out = nullptr;
    const uint64_t need = align_up(bytes ? bytes : 1, BLOCK_ALIGN);
    std::lock_guard<std::mutex> lk(_mtx);
    // first fit over the idle blocks of every chunk, smallest chunks first is not needed: address order
    decx::MemBlock* hit = nullptr;
    for (Chunk& c : _chunks) {
        for (decx::MemBlock* b = c.first; b != nullptr; b = b->next)
            if (b->idle && b->size >= need) { hit = b; break; }
        if (hit) break;
    }
    if (hit == nullptr) {
        // a new physical chunk of 2^k bytes, as the reference does (a 2 GiB matrix takes a 2^31 chunk)
        const uint64_t csize = pow2_at_least(need);
        void* base = nullptr;
        const int rc = g_raw_alloc(&base, size_t(csize));
        if (rc != 0 || base == nullptr) return rc != 0 ? rc : int(cudaErrorMemoryAllocation);
        decx::MemBlock* b = new decx::MemBlock;
        b->pool = this;
        b->ptr = static_cast<uint8_t*>(base);
        b->size = csize;
        b->chunk = int(_chunks.size());
        _chunks.push_back(Chunk{b->ptr, csize, b});
        hit = b;
    }
    if (hit->size > need) {   // split: [need | remainder]
        decx::MemBlock* rest = new decx::MemBlock;
        rest->pool = this;
        rest->ptr = hit->ptr + need;
        rest->size = hit->size - need;
        rest->chunk = hit->chunk;
        rest->prev = hit;
        rest->next = hit->next;
        if (hit->next) hit->next->prev = rest;
        hit->next = rest;
        hit->size = need;
    }
    hit->idle = false;
    hit->refcount = 1;
    *out = hit;
    return 0;
}

void decx::MemPool_D::register_reference(decx::MemBlock* b) {
    if (b == nullptr) return;
    std::lock_guard<std::mutex> lk(_mtx);
    ++b->refcount;
}

void decx::MemPool_D::merge_with_next(decx::MemBlock* b) {
    decx::MemBlock* n = b->next;
    b->size += n->size;
    b->next = n->next;
    if (n->next) n->next->prev = b;
    delete n;
}

void decx::MemPool_D::deallocate(decx::MemBlock* b) {
    if (b == nullptr) return;
    std::lock_guard<std::mutex> lk(_mtx);
    if (b->orphan) {                      // its chunk went back to CUDA in release(); only the record is left
        if (--b->refcount <= 0) delete b;
        return;
    }
    if (b->idle || --b->refcount > 0) return;
    b->idle = true;
    b->refcount = 0;
    if (b->next && b->next->idle) merge_with_next(b);
    if (b->prev && b->prev->idle) {
        decx::MemBlock* p = b->prev;
        merge_with_next(p);
    }
}

void decx::MemPool_D::release() {
    std::lock_guard<std::mutex> lk(_mtx);
    for (Chunk& c : _chunks) {
        for (decx::MemBlock* b = c.first; b != nullptr;) {
            decx::MemBlock* n = b->next;
            if (b->idle) {
                delete b;
            } else {
                // a matrix or scratch object still holds this block (the reference frees only the chunk memory
                // here, MemoryPool_D.cu:154-166, so releasing such an object later is harmless there): keep the
                // record so that a later deallocate() finds valid metadata; the last reference deletes it
                b->orphan = true;
                b->ptr = nullptr;
                b->size = 0;
                b->prev = b->next = nullptr;
                b->chunk = -1;
            }
            b = n;
        }
        g_raw_free(c.base);
    }
    _chunks.clear();
}

uint64_t decx::MemPool_D::bytes_reserved() const {
    std::lock_guard<std::mutex> lk(_mtx);
    uint64_t s = 0;
    for (const Chunk& c : _chunks) s += c.size;
    return s;
}

uint64_t decx::MemPool_D::bytes_in_use() const {
    std::lock_guard<std::mutex> lk(_mtx);
    uint64_t s = 0;
    for (const Chunk& c : _chunks)
        for (const decx::MemBlock* b = c.first; b; b = b->next)
            if (!b->idle) s += b->size;
    return s;
}

size_t decx::MemPool_D::chunk_count() const {
    std::lock_guard<std::mutex> lk(_mtx);
    return _chunks.size();
}

size_t decx::MemPool_D::idle_block_count() const {
    std::lock_guard<std::mutex> lk(_mtx);
    size_t n = 0;
    for (const Chunk& c : _chunks)
        for (const decx::MemBlock* b = c.first; b; b = b->next) n += b->idle ? 1 : 0;
    return n;
}

// blocks tile their chunk exactly, are 256-byte aligned, no two idle neighbours remain unmerged
bool decx::MemPool_D::check_invariants() const {
    std::lock_guard<std::mutex> lk(_mtx);
    for (const Chunk& c : _chunks) {
        const uint8_t* at = c.base;
        const decx::MemBlock* prev = nullptr;
        for (const decx::MemBlock* b = c.first; b; b = b->next) {
            if (b->ptr != at || b->prev != prev || b->size == 0) return false;
            if ((reinterpret_cast<uintptr_t>(b->ptr) - reinterpret_cast<uintptr_t>(c.base)) % BLOCK_ALIGN) return false;
            if (prev && prev->idle && b->idle) return false;
            if (b->idle != (b->refcount == 0)) return false;
            at += b->size;
            prev = b;
        }
        if (at != c.base + c.size) return false;
    }
    return true;
}

// ------------------------------------------------------------------------------------------------ decx::alloc
namespace {
int current_device() {
    int d = 0;
    cudaGetDevice(&d);
    return d;
}
}  // namespace

int decx::alloc::_device_malloc(decx::PtrInfo<void>* p, uint64_t bytes, bool set_zero, decx::cuda_stream* S) {
    decx::MemBlock* b = nullptr;
    const int rc = decx::MemPool_D::GetInstance(current_device())->allocate(bytes, &b);
    if (rc != 0) {
        p->block = nullptr;
        p->ptr = nullptr;
        return rc;
    }
    p->block = b;
    p->ptr = b->ptr;
    if (set_zero) {
        const cudaError_t e = S ? cudaMemsetAsync(p->ptr, 0, bytes, S->get_raw_stream_ref()) : cudaMemset(p->ptr, 0, bytes);
        if (e != cudaSuccess) {
            decx::alloc::_device_dealloc(p);      // nothing is handed out on failure
            return int(e);
        }
    }
    return 0;
}

int decx::alloc::_device_realloc(decx::PtrInfo<void>* p, uint64_t bytes, bool set_zero, decx::cuda_stream* S) {
    if (p->block != nullptr && !p->block->orphan && p->block->size >= bytes && p->block->refcount == 1) {
        if (set_zero) {
            const cudaError_t e = S ? cudaMemsetAsync(p->ptr, 0, bytes, S->get_raw_stream_ref()) : cudaMemset(p->ptr, 0, bytes);
            if (e != cudaSuccess) return int(e);
        }
        return 0;
    }
    decx::alloc::_device_dealloc(p);
    return decx::alloc::_device_malloc(p, bytes, set_zero, S);
}

void decx::alloc::_device_dealloc(decx::PtrInfo<void>* p) {
    if (p->block != nullptr) p->block->pool->deallocate(p->block);   // back to the pool (device) it came from
    p->block = nullptr;
    p->ptr = nullptr;
}

void decx::alloc::_device_malloc_same_place(decx::PtrInfo<void>* p) {
    if (p->block != nullptr) p->block->pool->register_reference(p->block);
}

// ------------------------------------------------------------------------------------------------ block-level interface
int decx::alloc::_alloc_D(decx::MemBlock** _ptr, size_t req_size) {
    if (_ptr == nullptr) return -1;
    return decx::MemPool_D::GetInstance(current_device())->allocate(req_size, _ptr) == 0 ? 0 : -1;
}

void decx::alloc::_alloc_D_same_place(decx::MemBlock** _ptr) {
    if (_ptr != nullptr && *_ptr != nullptr) (*_ptr)->pool->register_reference(*_ptr);
}

void decx::alloc::_dealloc_D(decx::MemBlock* _ptr) {
    if (_ptr != nullptr) _ptr->pool->deallocate(_ptr);
}

void decx::alloc::Memset_D(decx::MemBlock* _ptr, const size_t size, const int value, cudaStream_t* S) {
    if (_ptr == nullptr || _ptr->ptr == nullptr) return;
    const size_t n = size < _ptr->size ? size : size_t(_ptr->size);
    if (S != nullptr) cudaMemsetAsync(_ptr->ptr, value, n, *S);
    else cudaMemset(_ptr->ptr, value, n);
}
