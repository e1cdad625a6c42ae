// CPU-only unit tests of the C++ drop-in's host logic: ABI sizes, pitch rules, host matrix, half conversion,
// error handle, and the pooled device allocator driven through a fake raw allocator (no GPU is touched).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
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

int main() {
    test_abi();
    test_pitch_and_host_matrix();
    test_half();
    test_errors();
    test_pool();
    test_pool_release_under_live_objects();
    test_reconstruct_never_keeps_another_devices_block();
    if (g_fail == 0) std::printf("host_units: all checks passed\n");
    return g_fail == 0 ? 0 : 1;
}
