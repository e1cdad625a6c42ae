// extern "C" layer, third part: one host-matrix GEMM sharded over several GPUs of THIS process.
// Built on the public entry points (decxb200_gemm_fp16_fetch, decxb200_gemm_ex, decxb200_write_flag_async)
// plus copies and events of the CUDA runtime.  See include/decx_b200.h for the contract.
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/decx_b200.h"
#include "capi_shared.h"

using dxb_host::round_up;

namespace {

constexpr int MAX_MULTI = 16;
constexpr uint32_t MAX_PANELS = 16;

struct Plan {
    int world = 0;
    uint32_t M = 0, N = 0, K = 0;
    uint32_t row0[MAX_MULTI] = {0}, nrows[MAX_MULTI] = {0}, rb[MAX_MULTI] = {0};     // rows of A / D per device, block height
    uint32_t piece0[MAX_MULTI] = {0}, piece_rows[MAX_MULTI] = {0};                   // rows of B each device uploads
    uint32_t n_panels = 0, panel_end[MAX_PANELS] = {0};
    uint64_t ld_k = 0, ld_n = 0;                                                     // device pitches (elements)
    // arena offsets (bytes)
    uint64_t off_flags = 0, off_scratch = 0, off_b = 0, off_a[2] = {0, 0}, off_d[2] = {0, 0}, total = 0;
    uint32_t max_jobs = 0;
};

uint32_t block_rows(uint32_t rows) {
    if (rows <= 2048) return rows;
    // about eight steps of whole 256-row tiles, 1024 rows or more: what cannot overlap the copies is the last
    // block's GEMM and download
    uint32_t rb = uint32_t(round_up((uint64_t(rows) + 7) / 8, 256));
    if (rb < 1024) rb = 1024;
    return rb > rows ? rows : rb;
}

Plan make_plan(int world, uint32_t M, uint32_t N, uint32_t K) {
    Plan p;
    p.world = world;
    p.M = M; p.N = N; p.K = K;
    // rows of A in whole 256-row tiles, as evenly as they go
    const uint32_t tiles = (M + 255) / 256, per = (tiles + world - 1) / world;
    uint32_t max_rows = 0;
    for (int d = 0; d < world; ++d) {
        const uint64_t a = uint64_t(d) * per * 256, b = uint64_t(d + 1) * per * 256;
        p.row0[d] = uint32_t(a < M ? a : M);
        p.nrows[d] = uint32_t((b < M ? b : M) - p.row0[d]);
        p.rb[d] = block_rows(p.nrows[d]);
        if (p.nrows[d] > max_rows) max_rows = p.nrows[d];
    }
    // rows of B: one piece per device that has rows of A (the others take no part), multiples of 16 rows
    int active = 0;
    for (int d = 0; d < world; ++d) active += p.nrows[d] > 0;
    const uint32_t units = (K + 15) / 16;
    uint32_t r = 0, i = 0;
    for (int d = 0; d < world; ++d) {
        if (p.nrows[d] == 0) continue;
        const uint32_t u = units / active + (i < units % active ? 1 : 0);
        uint32_t n = u * 16;
        if (n > K - r) n = K - r;
        p.piece0[d] = r;
        p.piece_rows[d] = n;
        r += n;
        ++i;
    }
    // column panels: two 512-column tiles wide at first (early start), four afterwards, at most 16
    const uint32_t ctiles = (N + 511) / 512;
    uint32_t widths[64], nw = 0, left = ctiles;
    while (left > 0 && nw < 64) {
        uint32_t w = nw < 4 ? 2 : 4;
        if (w > left) w = left;
        widths[nw++] = w;
        left -= w;
    }
    while (nw > MAX_PANELS || left > 0) {                                  // very wide B: merge from the back
        if (nw < 2) break;
        widths[nw - 2] += widths[nw - 1] + left;
        left = 0;
        --nw;
    }
    uint32_t c = 0;
    for (uint32_t j = 0; j < nw; ++j) {
        c += widths[j] * 512;
        p.panel_end[j] = c < N ? c : N;
    }
    p.panel_end[nw - 1] = N;
    p.n_panels = nw;
    p.ld_k = round_up(uint64_t(K) * 2, 128) / 2;
    p.ld_n = round_up(uint64_t(N) * 2, 128) / 2;
    p.max_jobs = p.n_panels * uint32_t(world);
    uint64_t off = 0;
    auto take = [&](uint64_t bytes) { const uint64_t o = off; off += round_up(bytes, 256); return o; };
    p.off_flags = take(256);
    p.off_scratch = take(decxb200_fetch_scratch_bytes(p.max_jobs));
    p.off_b = take(uint64_t(K) * p.ld_n * 2);
    const uint32_t rbmax = block_rows(max_rows);
    for (int i2 = 0; i2 < 2; ++i2) {
        p.off_a[i2] = take(uint64_t(rbmax) * p.ld_k * 2);
        p.off_d[i2] = take(uint64_t(rbmax) * p.ld_n * 2);
    }
    p.total = off;
    return p;
}

struct DevCtx {
    bool ready = false;
    cudaStream_t h2d = nullptr, comp = nullptr, d2h = nullptr;
    cudaEvent_t ev_h2d[2] = {nullptr, nullptr}, ev_comp[2] = {nullptr, nullptr}, ev_d2h[2] = {nullptr, nullptr};
};
DevCtx g_ctx[64];
bool g_peer[64][64];
std::mutex g_mtx;

int dev_ctx(int dev, DevCtx*& out) {
    out = &g_ctx[dev];
    if (out->ready) return 0;
    cudaError_t e;
    for (cudaStream_t* s : {&out->h2d, &out->comp, &out->d2h})
        if ((e = cudaStreamCreateWithFlags(s, cudaStreamNonBlocking)) != cudaSuccess) return int(e);
    for (cudaEvent_t* ev : {&out->ev_h2d[0], &out->ev_h2d[1], &out->ev_comp[0], &out->ev_comp[1], &out->ev_d2h[0], &out->ev_d2h[1]})
        if ((e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming)) != cudaSuccess) return int(e);
    out->ready = true;
    return 0;
}

// every device of the set can read every other one's memory?  (enables it on first use)
bool enable_peers(const int* devices, int world) {
    for (int i = 0; i < world; ++i)
        for (int j = 0; j < world; ++j) {
            const int a = devices[i], b = devices[j];
            if (a == b || g_peer[a][b]) continue;
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, a, b) != cudaSuccess || !can) { cudaGetLastError(); return false; }
            if (cudaSetDevice(a) != cudaSuccess) return false;
            const cudaError_t e = cudaDeviceEnablePeerAccess(b, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return false; }
            cudaGetLastError();
            g_peer[a][b] = true;
        }
    return true;
}

}  // namespace

extern "C" {

size_t decxb200_gemm_host_multi_arena_bytes(int dtype, int n_devices, uint32_t M, uint32_t N, uint32_t K) {
    if (dtype != DECXB200_FP16 || n_devices < 1 || n_devices > MAX_MULTI || M == 0 || N == 0 || K == 0) return 0;
    return size_t(make_plan(n_devices, M, N, K).total);
}

int decxb200_gemm_host_multi_plan(int n_devices, uint32_t M, uint32_t N, uint32_t K, uint32_t* row0, uint32_t* nrows,
                                  uint32_t* block_rows_out, uint32_t* piece0, uint32_t* piece_rows, uint32_t* n_panels,
                                  uint32_t* panel_end) {
    if (n_devices < 1 || n_devices > MAX_MULTI || M == 0 || N == 0 || K == 0) return DECXB200_EINVAL;
    const Plan p = make_plan(n_devices, M, N, K);
    for (int d = 0; d < n_devices; ++d) {
        if (row0) row0[d] = p.row0[d];
        if (nrows) nrows[d] = p.nrows[d];
        if (block_rows_out) block_rows_out[d] = p.rb[d];
        if (piece0) piece0[d] = p.piece0[d];
        if (piece_rows) piece_rows[d] = p.piece_rows[d];
    }
    if (n_panels) *n_panels = p.n_panels;
    if (panel_end)
        for (uint32_t j = 0; j < p.n_panels; ++j) panel_end[j] = p.panel_end[j];
    return 0;
}

int decxb200_gemm_host_multi(int dtype, int n_devices, const int* devices, uint32_t M, uint32_t N, uint32_t K,
                             const void* A, uint64_t lda, const void* B, uint64_t ldb, void* D, uint64_t ldd,
                             void* const* arenas, size_t arena_bytes) {
    dxb_host::reset_launches();
    if (dtype != DECXB200_FP16) return DECXB200_EINVAL;
    if (n_devices < 1 || n_devices > MAX_MULTI || devices == nullptr || arenas == nullptr) return DECXB200_EINVAL;
    if (A == nullptr || B == nullptr || D == nullptr || M == 0 || N == 0 || K == 0 || lda < K || ldb < N || ldd < N)
        return DECXB200_EINVAL;
    if ((N % 8) != 0) return DECXB200_EALIGN;                     // courier copies move 16-byte units of a row
    const Plan pl = make_plan(n_devices, M, N, K);
    if (arena_bytes < pl.total) return DECXB200_EWORKSPACE;
    for (int d = 0; d < n_devices; ++d) {
        if (devices[d] < 0 || devices[d] >= 64) return DECXB200_EINVAL;
        for (int e2 = 0; e2 < d; ++e2)
            if (devices[e2] == devices[d]) return DECXB200_EINVAL;
        if (arenas[d] == nullptr || (reinterpret_cast<uintptr_t>(arenas[d]) & 255) != 0) return DECXB200_EWORKSPACE;
    }
    std::lock_guard<std::mutex> lk(g_mtx);                         // one multi-GPU call at a time per process
    int prev = 0;
    cudaGetDevice(&prev);
    int rc = 0;
    cudaError_t e = cudaSuccess;
#define MG_CUDA(call) do { e = (call); if (e != cudaSuccess) { rc = int(e); goto out; } } while (0)
#define MG_RC(call) do { rc = (call); if (rc != 0) goto out; } while (0)
    {
        int active = 0;
        for (int d = 0; d < n_devices; ++d) active += pl.nrows[d] > 0;
        // with peer access the devices complete each other's B over NVLink; without it each one uploads all of B
        const bool gather = active > 1 && enable_peers(devices, n_devices);
        DevCtx* cx[MAX_MULTI];
        auto at = [&](int d, uint64_t off) { return static_cast<uint8_t*>(arenas[d]) + off; };
        auto flags = [&](int d) { return reinterpret_cast<unsigned*>(at(d, pl.off_flags)); };      // ready[16], pub[16], status
        const unsigned epoch = 1;
        // 1. clean flags everywhere before anything can look at them
        for (int d = 0; d < n_devices; ++d) {
            if (pl.nrows[d] == 0) continue;
            MG_CUDA(cudaSetDevice(devices[d]));
            MG_RC(dev_ctx(devices[d], cx[d]));
            MG_CUDA(cudaMemsetAsync(flags(d), 0, 256, cx[d]->h2d));
        }
        for (int d = 0; d < n_devices; ++d)
            if (pl.nrows[d] > 0) { MG_CUDA(cudaSetDevice(devices[d])); MG_CUDA(cudaStreamSynchronize(cx[d]->h2d)); }
        // 2. uploads of B (each device its rows, panel by panel, flagged) and of the first block of A
        for (int d = 0; d < n_devices; ++d) {
            if (pl.nrows[d] == 0) continue;
            MG_CUDA(cudaSetDevice(devices[d]));
            const uint32_t r0 = gather ? pl.piece0[d] : 0, nr = gather ? pl.piece_rows[d] : K;
            uint32_t c0 = 0;
            for (uint32_t p = 0; p < pl.n_panels; ++p) {
                const uint32_t w = pl.panel_end[p] - c0;
                if (nr > 0)
                    MG_CUDA(cudaMemcpy2DAsync(at(d, pl.off_b) + (uint64_t(r0) * pl.ld_n + c0) * 2, pl.ld_n * 2,
                                              static_cast<const uint8_t*>(B) + (uint64_t(r0) * ldb + c0) * 2, ldb * 2,
                                              uint64_t(w) * 2, nr, cudaMemcpyHostToDevice, cx[d]->h2d));
                MG_RC(decxb200_write_flag_async(cx[d]->h2d, flags(d) + 16 + p, epoch));     // pub: my rows of panel p are here
                if (p == 0) {
                    // the first block of A goes right behind the first panel, so the first tiles can start early
                    const uint32_t rows = pl.rb[d] < pl.nrows[d] ? pl.rb[d] : pl.nrows[d];
                    MG_CUDA(cudaMemcpy2DAsync(at(d, pl.off_a[0]), pl.ld_k * 2,
                                              static_cast<const uint8_t*>(A) + uint64_t(pl.row0[d]) * lda * 2, lda * 2,
                                              uint64_t(K) * 2, rows, cudaMemcpyHostToDevice, cx[d]->h2d));
                    MG_CUDA(cudaEventRecord(cx[d]->ev_h2d[0], cx[d]->h2d));
                }
                c0 = pl.panel_end[p];
            }
        }
        // 3. row blocks: block 0 runs the kernel that also brings in the other devices' rows of B
        uint32_t max_steps = 0;
        for (int d = 0; d < n_devices; ++d)
            if (pl.nrows[d] > 0) {
                const uint32_t s = (pl.nrows[d] + pl.rb[d] - 1) / pl.rb[d];
                if (s > max_steps) max_steps = s;
            }
        for (uint32_t step = 0; step < max_steps; ++step) {
            for (int d = 0; d < n_devices; ++d) {
                if (pl.nrows[d] == 0) continue;
                const uint32_t blk0 = step * pl.rb[d];
                if (blk0 >= pl.nrows[d]) continue;
                const uint32_t rows = pl.nrows[d] - blk0 < pl.rb[d] ? pl.nrows[d] - blk0 : pl.rb[d];
                const int b = int(step & 1u);
                MG_CUDA(cudaSetDevice(devices[d]));
                if (step > 0) {
                    if (step >= 2) MG_CUDA(cudaStreamWaitEvent(cx[d]->h2d, cx[d]->ev_comp[b], 0));      // A staging free again
                    MG_CUDA(cudaMemcpy2DAsync(at(d, pl.off_a[b]), pl.ld_k * 2,
                                              static_cast<const uint8_t*>(A) + uint64_t(pl.row0[d] + blk0) * lda * 2, lda * 2,
                                              uint64_t(K) * 2, rows, cudaMemcpyHostToDevice, cx[d]->h2d));
                    MG_CUDA(cudaEventRecord(cx[d]->ev_h2d[b], cx[d]->h2d));
                }
                MG_CUDA(cudaStreamWaitEvent(cx[d]->comp, cx[d]->ev_h2d[b], 0));
                if (step >= 2) MG_CUDA(cudaStreamWaitEvent(cx[d]->comp, cx[d]->ev_d2h[b], 0));           // D staging drained
                unsigned* status = flags(d) + 32;
                if (step == 0) {
                    std::vector<decxb200_fetch_job> jobs;
                    uint32_t c0 = 0;
                    for (uint32_t p = 0; p < pl.n_panels; ++p) {
                        const uint32_t w = pl.panel_end[p] - c0;
                        // my own rows arrive by copy engine: wait for their flag, nothing to copy
                        jobs.push_back({nullptr, flags(d) + 16 + p, nullptr, nullptr, gather ? pl.piece0[d] : 0u, 0u, c0, w, p, 0u});
                        if (gather)
                            for (int k = 1; k < n_devices; ++k) {
                                const int h = (d + k) % n_devices;                                   // stagger the sources
                                if (pl.nrows[h] == 0 || pl.piece_rows[h] == 0) continue;
                                jobs.push_back({at(h, pl.off_b), flags(h) + 16 + p, nullptr, nullptr, pl.piece0[h], pl.piece_rows[h], c0, w, p, 0u});
                            }
                        c0 = pl.panel_end[p];
                    }
                    MG_RC(decxb200_gemm_fp16_fetch(cx[d]->comp, rows, N, K, at(d, pl.off_a[b]), pl.ld_k, at(d, pl.off_b), pl.ld_n,
                                                   at(d, pl.off_d[b]), pl.ld_n, status, pl.n_panels, pl.panel_end, flags(d),
                                                   flags(d) + 16, epoch, jobs.data(), uint32_t(jobs.size()),
                                                   at(d, pl.off_scratch), decxb200_fetch_scratch_bytes(pl.max_jobs), 0, 0));
                } else {
                    MG_RC(decxb200_gemm_ex(DECXB200_FP16, cx[d]->comp, rows, N, K, at(d, pl.off_a[b]), pl.ld_k, at(d, pl.off_b),
                                           pl.ld_n, nullptr, 0, at(d, pl.off_d[b]), pl.ld_n, nullptr, nullptr, nullptr, 0, status,
                                           0, 0));
                }
                MG_CUDA(cudaEventRecord(cx[d]->ev_comp[b], cx[d]->comp));
                MG_CUDA(cudaStreamWaitEvent(cx[d]->d2h, cx[d]->ev_comp[b], 0));
                MG_CUDA(cudaMemcpy2DAsync(static_cast<uint8_t*>(D) + uint64_t(pl.row0[d] + blk0) * ldd * 2, ldd * 2,
                                          at(d, pl.off_d[b]), pl.ld_n * 2, uint64_t(N) * 2, rows, cudaMemcpyDeviceToHost,
                                          cx[d]->d2h));
                MG_CUDA(cudaEventRecord(cx[d]->ev_d2h[b], cx[d]->d2h));
            }
        }
        // 4. finish: every stream of every device, then the status words
        for (int d = 0; d < n_devices; ++d) {
            if (pl.nrows[d] == 0) continue;
            MG_CUDA(cudaSetDevice(devices[d]));
            MG_CUDA(cudaStreamSynchronize(cx[d]->d2h));
            MG_CUDA(cudaStreamSynchronize(cx[d]->comp));
            MG_CUDA(cudaStreamSynchronize(cx[d]->h2d));
        }
        for (int d = 0; d < n_devices; ++d) {
            if (pl.nrows[d] == 0) continue;
            unsigned st = 0;
            MG_CUDA(cudaSetDevice(devices[d]));
            MG_CUDA(cudaMemcpy(&st, flags(d) + 32, sizeof(st), cudaMemcpyDeviceToHost));
            if (st != 0) { rc = DECXB200_EKERNEL; goto out; }
        }
    }
out:
#undef MG_CUDA
#undef MG_RC
    if (rc != 0) {
        // leave nothing in flight that still reads the caller's buffers
        for (int d = 0; d < n_devices; ++d)
            if (cudaSetDevice(devices[d]) == cudaSuccess) cudaDeviceSynchronize();
        cudaGetLastError();
    }
    cudaSetDevice(prev);
    return rc;
}

}  // extern "C"
