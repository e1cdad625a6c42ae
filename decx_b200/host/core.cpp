// Error handle, start-up calls, half conversion, resource manager.
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <thread>

#include "internal.h"

// ------------------------------------------------------------------------------------------------ errors
namespace {
de::DH g_last_error = {de::DECX_SUCCESS, "success: No error"};
std::mutex g_err_mtx;
}  // namespace

void decx::err::set(de::DH* handle, int code, const char* message) {
    std::lock_guard<std::mutex> lk(g_err_mtx);
    handle->error_type = code;
    std::strncpy(handle->error_string, message, sizeof(handle->error_string) - 1);
    handle->error_string[sizeof(handle->error_string) - 1] = '\0';
}
void decx::err::success(de::DH* handle) { decx::err::set(handle, de::DECX_SUCCESS, "success: No error"); }

de::DH* de::GetLastError() { return &g_last_error; }
void de::ResetLastError() { decx::err::success(&g_last_error); }

// ------------------------------------------------------------------------------------------------ init
namespace {
bool g_cuda_init = false;
cudaDeviceProp g_prop;
uint64_t g_cpu_concurrency = 1, g_hw_concurrency = 1;
}  // namespace

void de::InitCuda() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceProperties(&g_prop, dev) != cudaSuccess) {
        decx::err::set(de::GetLastError(), de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first");
        return;
    }
    g_cuda_init = true;
}
bool decx::cuda::_is_CUDA_init() { return g_cuda_init; }
const cudaDeviceProp& decx::cuda::_get_cuda_prop() { return g_prop; }

void de::InitCPUInfo() {
    g_hw_concurrency = std::thread::hardware_concurrency();
    if (g_hw_concurrency == 0) g_hw_concurrency = 1;
    g_cpu_concurrency = g_hw_concurrency;
}

void de::cpu::DecxSetThreadingNum(const uint64_t _thread_num) {
    g_cpu_concurrency = _thread_num < 1 ? 1 : _thread_num;
    if (_thread_num > g_hw_concurrency)
        decx::err::set(de::GetLastError(), de::CPU_HYPER_THREADING, "warning: Threading number exceeds the hardware concurrency");
    else
        decx::err::success(de::GetLastError());
}

void de::cuda::DECX_CUDA_exit() {
    decx::res::release_all();
    decx::cuda::release_stream_event_pools();
    int n = 0;
    if (cudaGetDeviceCount(&n) == cudaSuccess)
        for (int d = 0; d < n; ++d) decx::MemPool_D::GetInstance(d)->release();
}

// ------------------------------------------------------------------------------------------------ fp16 scalars
// (reference: srcs/common/FP16/float_half_convert.cu:33-45 uses the CUDA intrinsics on the host; this is the
// same IEEE round-to-nearest-even conversion written out)
de::Half de::Float2Half(const float& __x) {
    uint32_t x;
    std::memcpy(&x, &__x, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7FFFFFFFu;
    de::Half h;
    if (x >= 0x7F800000u) { h.val = uint16_t(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u : 0u)); return h; }
    if (x >= 0x477FF000u) { h.val = uint16_t(sign | 0x7C00u); return h; }
    if (x < 0x33000001u) { h.val = uint16_t(sign); return h; }
    const int32_t e = int32_t(x >> 23) - 127;
    const uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
    const int shift = e < -14 ? 13 + (-14 - e) : 13;
    const uint32_t hexp = e < -14 ? 0u : uint32_t(e + 15);
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    h.val = uint16_t(hexp == 0 ? (sign | q) : (sign | (((hexp - 1) << 10) + q)));
    return h;
}

float de::Half2Float(const de::Half& __x) {
    const uint16_t h = __x.val;
    const uint32_t sign = uint32_t(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            bits = sign | (uint32_t(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// ------------------------------------------------------------------------------------------------ resources
namespace {
std::mutex g_res_mtx;
std::vector<decx::ScratchResource*> g_resources;
std::condition_variable g_res_cv;
std::thread g_res_thread;
bool g_res_stop = false, g_res_started = false;

struct GenericResource {       // one ResourceCheckIn registration; ids are indices and are never reused
    void** exposed = nullptr;
    double lifespan = 0.0, last_used = 0.0;
    decx::res_release_fn release = nullptr;
    bool occupied = false, alive = false;
};
std::vector<GenericResource> g_generic;

void manager_loop() {
    std::unique_lock<std::mutex> lk(g_res_mtx);
    while (!g_res_stop) {
        g_res_cv.wait_for(lk, std::chrono::milliseconds(200));
        if (g_res_stop) break;
        const double now = decx::res::now_seconds();
        for (decx::ScratchResource* r : g_resources) r->collect_if_idle(now);
        for (GenericResource& g : g_generic) {
            if (!g.alive || g.occupied || g.exposed == nullptr || *g.exposed == nullptr) continue;
            if (now - g.last_used > g.lifespan) {
                if (g.release != nullptr) g.release(*g.exposed);
                *g.exposed = nullptr;
            }
        }
    }
}

void start_manager_locked() {
    if (!g_res_started) {
        g_res_started = true;
        g_res_thread = std::thread(manager_loop);
    }
}

struct ManagerGuard {   // stops the collector before static destruction tears the lists down
    ~ManagerGuard() {
        {
            std::lock_guard<std::mutex> lk(g_res_mtx);
            g_res_stop = true;
        }
        g_res_cv.notify_all();
        if (g_res_thread.joinable()) g_res_thread.join();
    }
} g_manager_guard;
}  // namespace

double decx::res::now_seconds() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

void decx::res::register_resource(decx::ScratchResource* r) {
    std::lock_guard<std::mutex> lk(g_res_mtx);
    g_resources.push_back(r);
    start_manager_locked();
}

uint64_t decx::ResourceCheckIn(void** exposed_ptr, const time_t lifespan_sec, decx::res_release_fn _decon) {
    std::lock_guard<std::mutex> lk(g_res_mtx);
    GenericResource g;
    g.exposed = exposed_ptr;
    g.lifespan = double(lifespan_sec);
    g.last_used = decx::res::now_seconds();
    g.release = _decon;
    g.alive = true;
    g_generic.push_back(g);
    start_manager_locked();
    return g_generic.size() - 1;
}

void decx::ResourceLock(const uint64_t res_id) {
    std::lock_guard<std::mutex> lk(g_res_mtx);
    if (res_id < g_generic.size()) g_generic[res_id].occupied = true;
}

void decx::ResourceUnlock(const uint64_t res_id) {
    std::lock_guard<std::mutex> lk(g_res_mtx);
    if (res_id < g_generic.size()) {
        g_generic[res_id].occupied = false;
        g_generic[res_id].last_used = decx::res::now_seconds();
    }
}

void decx::ResourceCheckOut(const uint64_t res_id) {
    std::lock_guard<std::mutex> lk(g_res_mtx);
    if (res_id >= g_generic.size() || !g_generic[res_id].alive) return;
    GenericResource& g = g_generic[res_id];
    if (g.exposed != nullptr && *g.exposed != nullptr) {
        if (g.release != nullptr) g.release(*g.exposed);
        *g.exposed = nullptr;
    }
    g.alive = false;
}

void decx::res::unregister_resource(decx::ScratchResource* r) {
    std::lock_guard<std::mutex> lk(g_res_mtx);
    for (size_t i = 0; i < g_resources.size(); ++i)
        if (g_resources[i] == r) { g_resources.erase(g_resources.begin() + i); break; }
}

void decx::res::release_all() {
    std::lock_guard<std::mutex> lk(g_res_mtx);
    for (decx::ScratchResource* r : g_resources) r->release_now();
}

decx::ScratchResource::ScratchResource(double lifespan_seconds) : _lifespan(lifespan_seconds) {
    decx::res::register_resource(this);
}
decx::ScratchResource::~ScratchResource() { decx::res::unregister_resource(this); }

void* decx::ScratchResource::lock(uint64_t bytes, int device) {
    _mtx.lock();
    if (_mem.ptr != nullptr && (_device != device || _bytes < bytes)) {
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur != _device) cudaSetDevice(_device);
        decx::alloc::_device_dealloc(&_mem);
        if (cur != _device) cudaSetDevice(cur);
        _bytes = 0;
    }
    if (_mem.ptr == nullptr && bytes > 0) {
        if (decx::alloc::_device_malloc(&_mem, bytes) != 0) {
            _mtx.unlock();
            return nullptr;
        }
        _bytes = bytes;
        _device = device;
    }
    _last_used = decx::res::now_seconds();
    return _mem.ptr;
}

void decx::ScratchResource::unlock() {
    _last_used = decx::res::now_seconds();
    _mtx.unlock();
}

void decx::ScratchResource::collect_if_idle(double now) {
    if (!_mtx.try_lock()) return;   // in use: not idle
    if (_mem.ptr != nullptr && now - _last_used > _lifespan) {
        int cur = 0;
        cudaGetDevice(&cur);
        cudaSetDevice(_device);
        decx::alloc::_device_dealloc(&_mem);
        cudaSetDevice(cur);
        _bytes = 0;
    }
    _mtx.unlock();
}

void decx::ScratchResource::release_now() {
    std::lock_guard<std::mutex> lk(_mtx);
    if (_mem.ptr != nullptr) {
        int cur = 0;
        cudaGetDevice(&cur);
        cudaSetDevice(_device);
        decx::alloc::_device_dealloc(&_mem);
        cudaSetDevice(cur);
        _bytes = 0;
    }
}
