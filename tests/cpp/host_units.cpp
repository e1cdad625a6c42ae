// CPU-only unit tests of the C++ drop-in's host logic: ABI sizes, pitch rules, host matrix, half conversion,
// error handle, and the pooled device allocator driven through a fake raw allocator (no GPU is touched).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <chrono>
#include <thread>
#include <vector>

#include "DECX.h"
#include "decx_b200/host/internal.h"

static int g_fail = 0;
#define CHECK(c) do { if (!(c)) { std::printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #c); ++g_fail; } } while (0)

// ---- fake device allocator: host memory, counts calls, can be told to fail
static int g_allocs = 0, g_frees = 0;
static bool g_fail_next = false;
static int fake_alloc(void** p, size_t bytes) {
    if (g_fail_next) { g_fail_next = false; *p = nullptr; return 2; }
    ++g_allocs;
    *p = std::aligned_alloc(256, bytes > (1u << 22) ? (1u << 22) : bytes);   // address space only: never dereferenced
    return *p ? 0 : 2;
}
static int fake_free(void* p) { ++g_frees; std::free(p); return 0; }

static void test_abi() {
    CHECK(sizeof(de::DH) == 104);
    CHECK(sizeof(de::Number) == 32);
    CHECK(sizeof(de::MatrixLayout) == 16);
    CHECK(sizeof(de::CPf) == 8 && alignof(de::CPf) == 8);
    CHECK(sizeof(de::Half) == 2);
    CHECK(sizeof(de::Point2D) == 8);
    CHECK(de::_FP32_ == 1 && de::_FP16_ == 3 && de::_COMPLEX_F32_ == 5);
    de::Number a(1.5f), h(de::Float2Half(0.25f)), c(de::CPf(1.f, -2.f));
    CHECK(a.Type() == de::_FP32_ && a.get_data<float>() == 1.5f);
    CHECK(h.Type() == de::_FP16_ && de::Half2Float(h.get_data<de::Half>()) == 0.25f);
    CHECK(c.Type() == de::_COMPLEX_F32_ && c.get_data<de::CPf>().image == -2.f);
}

static void test_pitch_and_host_matrix() {
    CHECK(decx::pitch_for(2053, 4, 32) == 2056);     // host, fp32: 8-float multiples
    CHECK(decx::pitch_for(2053, 4, 128) == 2080);    // device, fp32: 32-float multiples
    CHECK(decx::pitch_for(3001, 4, 128) == 3008);
    CHECK(decx::pitch_for(1013, 8, 128) == 1024);    // complex: 16-element multiples
    CHECK(decx::pitch_for(70, 2, 128) == 128);       // fp16: 64-element multiples
    de::Matrix& m = de::CreateMatrixRef(de::_FP32_, 13, 7);       // (type, WIDTH, HEIGHT)
    CHECK(m.Width() == 13 && m.Height() == 7 && m.Type() == de::_FP32_);
    *m.ptr<float>(6, 12) = 42.f;
    CHECK(*m.ptr<float>(0, 0) == 0.f);                              // zero-filled
    CHECK(m.ptr<float>(1, 0) - m.ptr<float>(0, 0) == 16);           // pitch: 13 floats -> 16
    CHECK(reinterpret_cast<uintptr_t>(m.ptr<float>(0, 0)) % 32 == 0);
    de::Matrix& s = de::CreateMatrixRef();
    s.SoftCopy(m);
    CHECK(s.Width() == 13 && *s.ptr<float>(6, 12) == 42.f && s.ptr<float>(0, 0) == m.ptr<float>(0, 0));
    m.release();
    CHECK(*s.ptr<float>(6, 12) == 42.f);                            // the soft copy keeps the storage alive
    s.release();
    de::Matrix& c = de::CreateMatrixRef(de::_COMPLEX_F32_, 5, 3);
    c.ptr<de::CPf>(2, 4)->image = 3.f;
    c.Reinterpret(de::_FP32_);
    CHECK(c.Width() == 10 && c.Type() == de::_FP32_ && *c.ptr<float>(2, 9) == 3.f);
    c.release();
}

static void test_half() {
    const float xs[] = {0.f, -0.f, 1.f, -2.5f, 65504.f, 65520.f, 1e-8f, 5.9604645e-8f, 6.1e-5f, 0.1f, 3.14159f, 1e6f};
    for (float x : xs) {
        const de::Half h = de::Float2Half(x);
        const float back = de::Half2Float(h);
        if (std::fabs(x) > 65519.f) CHECK(std::isinf(back));
        else if (std::fabs(x) < 2.98e-8f) CHECK(back == 0.f);
        else CHECK(std::fabs(back - x) <= std::fabs(x) * 0.0009766f + 3e-8f);
    }
    CHECK(de::Float2Half(1.0f).val == 0x3C00 && de::Float2Half(-2.0f).val == 0xC000);
    CHECK(de::Float2Half(1.00048828125f).val == 0x3C00);           // tie rounds to even
    CHECK(de::Float2Half(1.00146484375f).val == 0x3C02);
}

static void test_errors() {
    de::ResetLastError();
    CHECK(de::GetLastError()->error_type == de::DECX_SUCCESS);
    // nothing was initialised: the GEMM entry points must say so and do nothing
    de::Matrix& a = de::CreateMatrixRef(de::_FP32_, 4, 4);
    de::Matrix& b = de::CreateMatrixRef(de::_FP32_, 4, 4);
    de::Matrix& d = de::CreateMatrixRef();
    de::blas::cuda::GEMM(a, b, d);
    CHECK(de::GetLastError()->error_type == de::DECX_FAIL_CUDA_not_init);
    CHECK(std::strlen(de::GetLastError()->error_string) > 5);
    de::ResetLastError();
    de::InitCPUInfo();
    de::cpu::DecxSetThreadingNum(1u << 20);
    CHECK(de::GetLastError()->error_type == de::CPU_HYPER_THREADING);
    de::cpu::DecxSetThreadingNum(1);
    CHECK(de::GetLastError()->error_type == de::DECX_SUCCESS);
}

static void test_pool() {
    decx::MemPool_D::set_raw_allocator(fake_alloc, fake_free);
    decx::MemPool_D* pool = decx::MemPool_D::GetInstance(63);       // an ordinal nothing else uses
    decx::MemBlock *a, *b, *c, *d;
    CHECK(pool->allocate(1000, &a) == 0 && a->size == 1024);        // rounded to 256
    CHECK(a->pool == pool);                                         // a block remembers where it goes back to
    CHECK(pool->chunk_count() == 1 && pool->bytes_reserved() == (1u << 20) && g_allocs == 1);
    CHECK(pool->allocate(300000, &b) == 0 && pool->allocate(5, &c) == 0);
    CHECK(g_allocs == 1);                                           // carved from the same chunk
    CHECK(b->ptr == a->ptr + 1024 && c->ptr == b->ptr + b->size);
    CHECK(reinterpret_cast<uintptr_t>(c->ptr) % 256 == 0);
    CHECK(pool->check_invariants());
    pool->deallocate(b);                                            // hole in the middle
    CHECK(pool->idle_block_count() == 2 && pool->check_invariants());
    CHECK(pool->allocate(200000, &d) == 0 && d->ptr == a->ptr + 1024);   // first fit reuses the hole
    pool->register_reference(d);
    pool->deallocate(d);
    CHECK(!d->idle);                                                // still referenced once
    pool->deallocate(d);
    pool->deallocate(a);
    pool->deallocate(c);
    CHECK(pool->idle_block_count() == 1 && pool->bytes_in_use() == 0 && pool->check_invariants());   // all merged
    // a request larger than any chunk takes a new power-of-two chunk
    CHECK(pool->allocate((3u << 20) + 1, &a) == 0 && pool->chunk_count() == 2 && pool->bytes_reserved() == (1u << 20) + (4u << 20));
    // raw allocator failure surfaces as an error code, nothing is leaked or corrupted
    g_fail_next = true;
    CHECK(pool->allocate(64u << 20, &b) != 0 && b == nullptr && pool->check_invariants());
    pool->deallocate(a);
    // random churn against a shadow model
    std::vector<decx::MemBlock*> live;
    uint32_t seed = 12345;
    for (int i = 0; i < 4000; ++i) {
        seed = seed * 1664525u + 1013904223u;
        if (live.size() < 40 && (seed >> 16) % 3 != 0) {
            decx::MemBlock* x;
            CHECK(pool->allocate(1 + (seed >> 8) % 200000, &x) == 0);
            for (decx::MemBlock* o : live) CHECK(x->ptr + x->size <= o->ptr || o->ptr + o->size <= x->ptr);
            live.push_back(x);
        } else if (!live.empty()) {
            const size_t k = (seed >> 12) % live.size();
            pool->deallocate(live[k]);
            live.erase(live.begin() + k);
        }
    }
    CHECK(pool->check_invariants());
    for (decx::MemBlock* o : live) pool->deallocate(o);
    CHECK(pool->bytes_in_use() == 0 && pool->idle_block_count() == pool->chunk_count());
    const int chunks = int(pool->chunk_count());
    pool->release();
    CHECK(g_frees == chunks && pool->chunk_count() == 0 && pool->bytes_reserved() == 0);
    decx::MemPool_D::set_raw_allocator(nullptr, nullptr);
}

// The pool is released (DECX_CUDA_exit) while objects still hold blocks: their later release / re-shape must
// not touch freed metadata, and must never hand the stale memory out again.
static void test_pool_release_under_live_objects() {
    decx::MemPool_D::set_raw_allocator(fake_alloc, fake_free);
    decx::MemPool_D* pool = decx::MemPool_D::GetInstance(62);
    decx::PtrInfo<void> a, b;
    decx::MemBlock* blk = nullptr;
    CHECK(pool->allocate(4096, &blk) == 0);
    a.block = blk; a.ptr = blk->ptr;
    CHECK(pool->allocate(8192, &blk) == 0);
    b.block = blk; b.ptr = blk->ptr;
    decx::alloc::_device_malloc_same_place(&b);             // two holders of b
    pool->release();
    CHECK(pool->chunk_count() == 0 && pool->bytes_reserved() == 0);
    CHECK(a.block->orphan && b.block->orphan && a.block->ptr == nullptr);
    decx::alloc::_device_dealloc(&a);                       // deletes the orphan record
    CHECK(a.block == nullptr);
    decx::PtrInfo<void> b2 = b;
    decx::alloc::_device_dealloc(&b);                       // first holder
    // a matrix that still holds the orphan must not reuse it when re-shaped
    decx::_GPU_Matrix m;
    m.Mat = b2;
    m._init = true;
    m._device = 62;
    m.type = de::_FP32_;
    m._layout.width = 8; m._layout.height = 8; m._layout.pitch = 32; m._layout._single_element_size = 4;
    m.re_construct(de::_FP32_, 8, 8);                       // same shape: used to return early and keep the dead block
    CHECK(m.Mat.block == nullptr || !m.Mat.block->orphan);
    m.release();
    CHECK(pool->check_invariants());
    decx::MemPool_D::GetInstance(0)->release();
    decx::MemPool_D::set_raw_allocator(nullptr, nullptr);
}

// dst was built on another GPU than the one the GEMM is about to run on: its block must go back to ITS pool and
// must not be written through by a kernel of the current device.
static void test_reconstruct_never_keeps_another_devices_block() {
    decx::MemPool_D::set_raw_allocator(fake_alloc, fake_free);
    decx::MemPool_D* other = decx::MemPool_D::GetInstance(61);
    decx::MemBlock* blk = nullptr;
    CHECK(other->allocate(1 << 16, &blk) == 0);
    decx::_GPU_Matrix m;
    m.Mat.block = blk; m.Mat.ptr = blk->ptr;
    m._init = true;
    m._device = 61;
    m.type = de::_FP32_;
    m._layout.width = 64; m._layout.height = 64; m._layout.pitch = 64; m._layout._single_element_size = 4;
    m.total_bytes = 64 * 64 * 4;
    CHECK(other->bytes_in_use() == (1u << 16));
    m.re_construct(de::_FP32_, 64, 64);                     // current device is 0 (or none): not pool 61
    CHECK(other->bytes_in_use() == 0);                      // the old block went home
    CHECK(m.Mat.block == nullptr || m.Mat.block->pool != other);
    m.release();
    other->release();
    decx::MemPool_D::GetInstance(0)->release();
    decx::MemPool_D::set_raw_allocator(nullptr, nullptr);
}

// ------------------------------------------------------------------------------------------------ stream / event pools
static int g_fake_dev = 0, g_streams_made = 0, g_streams_gone = 0, g_events_made = 0, g_events_gone = 0;
static int fake_stream_create(cudaStream_t* s, unsigned) { *s = reinterpret_cast<cudaStream_t>(uintptr_t(0x1000 + ++g_streams_made)); return 0; }
static int fake_stream_destroy(cudaStream_t) { ++g_streams_gone; return 0; }
static int fake_event_create(cudaEvent_t* e, unsigned) { *e = reinterpret_cast<cudaEvent_t>(uintptr_t(0x2000 + ++g_events_made)); return 0; }
static int fake_event_destroy(cudaEvent_t) { ++g_events_gone; return 0; }
static int fake_current_device() { return g_fake_dev; }

static void test_stream_event_pools() {
    const decx::cuda::RawHooks hooks = {fake_stream_create, fake_stream_destroy, fake_event_create, fake_event_destroy, fake_current_device};
    decx::cuda::set_raw_hooks(&hooks);
    decx::cuda_stream* a = decx::cuda::get_cuda_stream_ptr(1);
    decx::cuda_stream* b = decx::cuda::get_cuda_stream_ptr(1);
    CHECK(a != nullptr && b != nullptr && a != b && a->_is_occupied && decx::cuda::pooled_stream_count() == 2);
    a->detach();
    decx::cuda_stream* c = decx::cuda::get_cuda_stream_ptr(1);
    CHECK(c == a && g_streams_made == 2);                            // an idle stream with the same flag is reused
    decx::cuda_stream* d = decx::cuda::get_cuda_stream_ptr(0);
    CHECK(d != a && d != b && d->_flag == 0 && g_streams_made == 3); // another flag: a new stream
    c->detach();
    g_fake_dev = 1;
    decx::cuda_stream* e = decx::cuda::get_cuda_stream_ptr(1);
    CHECK(e != a && e->_device == 1 && g_streams_made == 4);         // never a stream of another device
    g_fake_dev = 0;
    decx::cuda_stream& r = decx::cuda::get_cuda_stream_ref(1);
    CHECK(&r == a);                                                  // the reference form draws from the same pool
    decx::cuda_event* e1 = decx::cuda::get_cuda_event_ptr(2);
    e1->detach();
    decx::cuda_event* e2 = decx::cuda::get_cuda_event_ptr(2);
    CHECK(e1 == e2 && g_events_made == 1 && decx::cuda::pooled_event_count() == 1);
    decx::cuda::release_stream_event_pools();
    CHECK(g_streams_gone == 4 && g_events_gone == 1 && decx::cuda::pooled_stream_count() == 0);
    decx::cuda::set_raw_hooks(nullptr);
}

// ------------------------------------------------------------------------------------------------ resource lifespans
static int g_released = 0;
static void release_int(void* p) { delete static_cast<int*>(p); ++g_released; }

static void sleep_ms(int ms) { std::this_thread::sleep_for(std::chrono::milliseconds(ms)); }

static void test_resource_lifespans() {
    // generic resources (the reference's ResourceCheckIn family): collected only when unlocked and idle
    void* obj = new int(7);
    const uint64_t id = decx::ResourceCheckIn(&obj, 1, release_int);
    decx::ResourceLock(id);
    sleep_ms(1600);
    CHECK(obj != nullptr && g_released == 0);                        // in use: survives its lifespan
    decx::ResourceUnlock(id);                                        // idle clock restarts here
    sleep_ms(400);
    decx::ResourceLock(id);                                          // users look at the object only while it is locked
    CHECK(obj != nullptr);
    decx::ResourceUnlock(id);
    sleep_ms(1800);
    decx::ResourceLock(id);
    CHECK(obj == nullptr && g_released == 1);                        // idle for more than 1 s: released, pointer cleared
    decx::ResourceUnlock(id);
    void* obj2 = new int(8);
    const uint64_t id2 = decx::ResourceCheckIn(&obj2, 100, release_int);
    decx::ResourceCheckOut(id2);
    CHECK(obj2 == nullptr && g_released == 2);                       // check-out releases at once
    decx::ResourceCheckOut(id2);                                     // and is idempotent
    CHECK(g_released == 2);

    // the GEMM workspace cache: a block of the device pool goes back after its lifespan
    decx::MemPool_D::set_raw_allocator(fake_alloc, fake_free);
    decx::MemPool_D* pool = decx::MemPool_D::GetInstance(0);         // CPU run: cudaGetDevice fails, ordinal 0 is used
    {
        decx::ScratchResource cache(0.2);
        void* p = cache.lock(5000, 0);
        CHECK(p != nullptr && pool->bytes_in_use() >= 5000 && cache.capacity() == 5000);   // capacity(): only while locked
        sleep_ms(700);
        CHECK(pool->bytes_in_use() >= 5000);                         // locked: the collector must not take it
        cache.unlock();
        void* q = cache.lock(4000, 0);
        CHECK(q == p);                                               // still cached, large enough: same block
        cache.unlock();
        sleep_ms(900);
        CHECK(pool->bytes_in_use() == 0);                            // idle > 0.2 s: back in the pool
        void* r = cache.lock(6000, 0);
        CHECK(r != nullptr && cache.capacity() == 6000);             // rebuilt on next use
        cache.unlock();
        cache.release_now();
        CHECK(pool->bytes_in_use() == 0);
    }
    pool->release();
    decx::MemPool_D::set_raw_allocator(nullptr, nullptr);
}

static void test_block_level_allocator() {
    decx::MemPool_D::set_raw_allocator(fake_alloc, fake_free);
    decx::MemPool_D* pool = decx::MemPool_D::GetInstance(0);
    decx::MemBlock* b = nullptr;
    CHECK(decx::alloc::_alloc_D(&b, 3000) == 0 && b != nullptr && b->size == 3072);
    decx::alloc::_alloc_D_same_place(&b);
    decx::alloc::_dealloc_D(b);
    CHECK(pool->bytes_in_use() == 3072);                             // one holder left
    decx::alloc::_dealloc_D(b);
    CHECK(pool->bytes_in_use() == 0);
    pool->release();
    decx::MemPool_D::set_raw_allocator(nullptr, nullptr);
}

static void test_vectors() {
    de::Vector& v = de::CreateVectorRef(de::_FP32_, 13);
    CHECK(v.Len() == 13 && v.Type() == de::_FP32_);
    decx::_Vector* iv = dynamic_cast<decx::_Vector*>(&v);
    CHECK(iv != nullptr && iv->_length == 16 && iv->total_bytes == 64 && reinterpret_cast<uintptr_t>(iv->data) % 64 == 0);
    for (int i = 0; i < 13; ++i) CHECK(*v.ptr<float>(i) == 0.f);
    *v.ptr<float>(12) = 5.f;
    de::Vector& w = de::CreateVectorRef();
    w.SoftCopy(v);
    CHECK(w.Len() == 13 && *w.ptr<float>(12) == 5.f);
    v.release();
    CHECK(*w.ptr<float>(12) == 5.f);                                 // shared storage outlives the first holder
    w.Reinterpret(de::_FP16_);
    CHECK(w.Len() == 26 && w.Type() == de::_FP16_);
    w.release();
    // slot order of the public interface (Len, release, SoftCopy, Type, Reinterpret)
    de::Vector* p = de::CreateVectorPtr(de::_FP16_, 4);
    void** vt = *reinterpret_cast<void***>(p);
    typedef size_t (*len_fn)(const de::Vector*);
    CHECK(reinterpret_cast<len_fn>(vt[0])(p) == 4);
    typedef de::_DATA_TYPES_FLAGS_ (*type_fn)(const de::Vector*);
    CHECK(reinterpret_cast<type_fn>(vt[3])(p) == de::_FP16_);
    p->release();
}

static void test_tensors() {
    // layouts: channels innermost, depth padded to 16 bytes, width to 4 (host) / 8 (device) columns
    CHECK(sizeof(de::Point3D) == 16);
    de::TensorLayout l;
    decx::tensor_layout(l, de::_FP32_, 13, 7, 3, 4);
    CHECK(l.dpitch == 4 && l.wpitch == 16 && l.dp_x_wp == 64 && l._single_element_size == 4);
    CHECK(l.plane[0] == 91 && l.plane[1] == 39 && l.plane[2] == 21);
    decx::tensor_layout(l, de::_FP32_, 13, 7, 3, 8);
    CHECK(l.dpitch == 4 && l.wpitch == 16);
    decx::tensor_layout(l, de::_FP32_, 17, 7, 9, 8);
    CHECK(l.dpitch == 12 && l.wpitch == 24);
    decx::tensor_layout(l, de::_FP16_, 5, 2, 9, 4);
    CHECK(l.dpitch == 16 && l.wpitch == 8);

    de::Tensor& t = de::CreateTensorRef(de::_FP32_, 13, 7, 3);        // (type, WIDTH, HEIGHT, DEPTH)
    CHECK(t.Width() == 13 && t.Height() == 7 && t.Depth() == 3 && t.Type() == de::_FP32_);
    CHECK(*t.ptr<float>(6, 12, 2) == 0.f);                             // zero-filled; ptr(row, column, channel)
    CHECK(t.ptr<float>(0, 1, 0) - t.ptr<float>(0, 0, 0) == 4);         // dpitch
    CHECK(t.ptr<float>(1, 0, 0) - t.ptr<float>(0, 0, 0) == 64);        // dp_x_wp
    *t.ptr<float>(6, 12, 2) = 7.f;
    de::Tensor& u = de::CreateTensorRef();
    u.SoftCopy(t);
    t.release();
    CHECK(u.Width() == 13 && *u.ptr<float>(6, 12, 2) == 7.f);         // shared storage outlives the first holder
    u.release();

    // host tensor array: tensors back to back; a slice is a view that keeps the storage alive
    de::TensorArray& a = de::CreateTensorArrayRef(de::_FP32_, 5, 3, 6, 4);
    CHECK(a.Width() == 5 && a.Height() == 3 && a.Depth() == 6 && a.TensorNum() == 4);
    CHECK(a.ptr<float>(0, 0, 0, 1) - a.ptr<float>(0, 0, 0, 0) == 3 * 8 * 8);     // gap = height * wpitch * dpitch
    *a.ptr<float>(2, 4, 5, 3) = 9.f;
    de::Tensor& sl = de::CreateTensorRef();
    CHECK(a.Extract_SoftCopy(3, sl).error_type == de::DECX_SUCCESS);
    CHECK(sl.Width() == 5 && sl.Depth() == 6 && sl.ptr<float>(0, 0, 0) == a.ptr<float>(0, 0, 0, 3));
    CHECK(a.Extract_SoftCopy(4, sl).error_type == de::DECX_FAIL_INVALID_PARAM);
    a.release();
    CHECK(*sl.ptr<float>(2, 4, 5) == 9.f);                             // the view outlives the array
    sl.release();

    // virtual slot order of the public interfaces
    de::TensorArray* pa = de::CreateTensorArrayPtr(de::_FP32_, 2, 2, 4, 3);
    void** vt = *reinterpret_cast<void***>(pa);
    typedef uint32_t (*u32_fn)(const void*);
    CHECK(reinterpret_cast<u32_fn>(vt[0])(pa) == 2 && reinterpret_cast<u32_fn>(vt[2])(pa) == 4 &&
          reinterpret_cast<u32_fn>(vt[3])(pa) == 3);                   // Width, Depth, TensorNum
    pa->release();

    // device tensor array on the fake allocator (no zero-fill, nothing dereferenced): slices share the block
    decx::MemPool_D::set_raw_allocator(fake_alloc, fake_free);
    decx::MemPool_D* pool = decx::MemPool_D::GetInstance(0);
    {
        decx::_GPU_TensorArray arr;
        arr.type = de::_FP32_;
        arr.tensor_num = 3;
        decx::tensor_layout(arr._layout, de::_FP32_, 5, 5, 16, 8);
        arr._gap = arr._layout.dp_x_wp * 5;
        arr.total_bytes = arr._gap * 3 * 4;
        arr._device = 0;
        CHECK(decx::alloc::_device_malloc(&arr.TensArr, arr.total_bytes, false) == 0);
        arr._init = true;
        CHECK(arr._gap == 5 * 8 * 16 && arr.Width() == 5 && arr.TensorNum() == 3);
        decx::_GPU_Tensor s1, s2;
        CHECK(arr.Extract_SoftCopy(1, s1).error_type == de::DECX_SUCCESS);
        CHECK(arr.Extract_SoftCopy(2, s2).error_type == de::DECX_SUCCESS);
        CHECK(arr.Extract_SoftCopy(3, s2).error_type == de::DECX_FAIL_INVALID_PARAM);
        CHECK(static_cast<uint8_t*>(s1.Tens.ptr) - static_cast<uint8_t*>(arr.TensArr.ptr) == int64_t(arr._gap * 4));
        CHECK(s1.Tens.block == arr.TensArr.block && arr.TensArr.block->refcount == 3);
        CHECK(s1.Width() == 5 && s1.Depth() == 16 && s1._layout.wpitch == 8);
        const uint64_t used = pool->bytes_in_use();
        arr.release();
        CHECK(pool->bytes_in_use() == used);                           // the slices keep the block
        // re_construct of a slice must not write into the array's block: it drops the share and would allocate
        s1.release();
        CHECK(pool->bytes_in_use() == used);
        s2.release();
        CHECK(pool->bytes_in_use() == 0);
    }
    pool->release();
    decx::MemPool_D::set_raw_allocator(nullptr, nullptr);

    // the API refuses to run before de::InitCuda
    de::GPU_Tensor& gs = de::CreateGPUTensorRef();
    de::GPU_TensorArray& gk = de::CreateGPUTensorArrayRef();
    de::GPU_Tensor& gd = de::CreateGPUTensorRef();
    CHECK(de::nn::cuda::Conv2D(gs, gk, gd, de::Point2D(1, 1), de::_EXTEND_CONSTANT_).error_type == de::DECX_FAIL_CUDA_not_init);
    de::Tensor& ht = de::CreateTensorRef(de::_FP32_, 2, 2, 4);
    CHECK(de::Memcpy(ht, gs, de::Point3D(0, 0, 0), de::Point3D(0, 0, 0), de::Point3D(4, 2, 2), de::DECX_MEMCPY_H2D).error_type ==
          de::DECX_FAIL_CUDA_not_init);
    ht.release();
}

int main() {
    test_abi();
    test_pitch_and_host_matrix();
    test_half();
    test_errors();
    test_pool();
    test_pool_release_under_live_objects();
    test_reconstruct_never_keeps_another_devices_block();
    test_stream_event_pools();
    test_block_level_allocator();
    test_vectors();
    test_resource_lifespans();
    test_tensors();
    if (g_fail == 0) std::printf("host_units: all checks passed\n");
    return g_fail == 0 ? 0 : 1;
}
