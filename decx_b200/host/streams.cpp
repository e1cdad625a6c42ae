// Stream and event pools: see internal.h.  One mutex guards both pools; objects are never destroyed
// before release_stream_event_pools(), so the pointers handed out stay valid.
#include <deque>

#include "internal.h"

namespace {
std::mutex g_mtx;
std::deque<decx::cuda_stream> g_streams;   // deque: growth keeps addresses of existing elements
std::deque<decx::cuda_event> g_events;

int current_device() {
    int d = 0;
    cudaGetDevice(&d);
    return d;
}

// creation / destruction go through these so that the pools can be unit-tested without a GPU
int real_stream_create(cudaStream_t* s, unsigned flag) { return int(cudaStreamCreateWithFlags(s, flag)); }
int real_stream_destroy(cudaStream_t s) { return int(cudaStreamDestroy(s)); }
int real_event_create(cudaEvent_t* e, unsigned flag) { return int(cudaEventCreateWithFlags(e, flag)); }
int real_event_destroy(cudaEvent_t e) { return int(cudaEventDestroy(e)); }
decx::cuda::RawHooks g_hooks = {real_stream_create, real_stream_destroy, real_event_create, real_event_destroy, nullptr};
}  // namespace

void decx::cuda::set_raw_hooks(const decx::cuda::RawHooks* hooks) {
    std::lock_guard<std::mutex> lk(g_mtx);
    if (hooks == nullptr) g_hooks = {real_stream_create, real_stream_destroy, real_event_create, real_event_destroy, nullptr};
    else g_hooks = *hooks;
}

void decx::cuda_stream::synchronize() { cudaStreamSynchronize(_S); }
void decx::cuda_stream::release() {
    if (_S != nullptr) g_hooks.stream_destroy(_S);
    _S = nullptr;
}
void decx::cuda_event::synchronize() { cudaEventSynchronize(_E); }
void decx::cuda_event::event_record(decx::cuda_stream* attached_stream) {
    cudaEventRecord(_E, attached_stream->get_raw_stream_ref());
}
void decx::cuda_event::release() {
    if (_E != nullptr) g_hooks.event_destroy(_E);
    _E = nullptr;
}

decx::cuda_stream* decx::cuda::get_cuda_stream_ptr(const int flag) {
    const int dev = g_hooks.current_device ? g_hooks.current_device() : current_device();
    std::lock_guard<std::mutex> lk(g_mtx);
    for (decx::cuda_stream& s : g_streams)
        if (!s._is_occupied && s._S != nullptr && s._flag == unsigned(flag) && s._device == dev) {
            s.attach();
            return &s;
        }
    cudaStream_t raw = nullptr;
    if (g_hooks.stream_create(&raw, unsigned(flag)) != 0) return nullptr;
    g_streams.emplace_back();
    decx::cuda_stream& s = g_streams.back();
    s._S = raw;
    s._flag = unsigned(flag);
    s._device = dev;
    s.attach();
    return &s;
}

decx::cuda_event* decx::cuda::get_cuda_event_ptr(const int flag) {
    const int dev = g_hooks.current_device ? g_hooks.current_device() : current_device();
    std::lock_guard<std::mutex> lk(g_mtx);
    for (decx::cuda_event& e : g_events)
        if (!e._is_occupied && e._E != nullptr && e._flag == unsigned(flag) && e._device == dev) {
            e.attach();
            return &e;
        }
    cudaEvent_t raw = nullptr;
    if (g_hooks.event_create(&raw, unsigned(flag)) != 0) return nullptr;
    g_events.emplace_back();
    decx::cuda_event& e = g_events.back();
    e._E = raw;
    e._flag = unsigned(flag);
    e._device = dev;
    e.attach();
    return &e;
}

void decx::cuda::release_stream_event_pools() {
    std::lock_guard<std::mutex> lk(g_mtx);
    for (decx::cuda_stream& s : g_streams) s.release();
    for (decx::cuda_event& e : g_events) e.release();
    g_streams.clear();
    g_events.clear();
}

size_t decx::cuda::pooled_stream_count() {
    std::lock_guard<std::mutex> lk(g_mtx);
    return g_streams.size();
}

size_t decx::cuda::pooled_event_count() {
    std::lock_guard<std::mutex> lk(g_mtx);
    return g_events.size();
}

decx::cuda_stream& decx::cuda::get_cuda_stream_ref(const int flag) {
    static decx::cuda_stream none;
    decx::cuda_stream* s = decx::cuda::get_cuda_stream_ptr(flag);
    return s != nullptr ? *s : none;
}

decx::cuda_event& decx::cuda::get_cuda_event_ref(const int flag) {
    static decx::cuda_event none;
    decx::cuda_event* e = decx::cuda::get_cuda_event_ptr(flag);
    return e != nullptr ? *e : none;
}
