// extern "C" layer of the B200 GEMM path: argument checks, tensor-map encoding,
// workspace carving, pre-pass and GEMM launches.  See include/decx_b200.h.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/decx_b200.h"
#include "capi_shared.h"
#include "gemm_sm100.cuh"
#include "prepass.cuh"

namespace dxb_host {
thread_local int t_launches = 0;
void count_launch(int n) { t_launches += n; }
void reset_launches() { t_launches = 0; }
}  // namespace dxb_host
using dxb_host::t_launches;

namespace {

using namespace dxb;
using dxb_host::round_up;
using dxb_host::aligned16;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library carries no link
// dependency on libcuda and still loads (without being able to compute) on a GPU-less host.
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

constexpr int MAX_DEVICES = 64;
struct DeviceInfo {
    unsigned ticket_base = 0;   // next starting value of the kernels' tile-barrier ticket counter
    int sm_count = 0;
    bool attr_set[2][2][2][6] = {};
};
DeviceInfo g_dev[MAX_DEVICES];
std::mutex g_dev_mutex;

thread_local int t_variant = 0;    // KIND*100 + CTAS*10 + NACC of the last GEMM kernel this thread launched


// Encoded tensor maps are cached per thread, keyed by everything that goes into them (base address, extents,
// pitch, box, swizzle, rank): a program that multiplies the same matrices again -- a training loop, the row blocks
// of the host-pointer path, a benchmark -- pays for cuTensorMapEncodeTiled once.  A map only DESCRIBES memory, so a
// stale entry for a freed and re-allocated address is still correct for the same key.
struct MapKey {
    const void* base; uint64_t rows, cols, ld; uint32_t b0, b1, b2; int f16, swizzle, rank;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && b0 == o.b0 && b1 == o.b1 && b2 == o.b2 &&
               f16 == o.f16 && swizzle == o.swizzle && rank == o.rank;
    }
};
struct MapCache {
    static constexpr int N = 48;
    MapKey key[N];
    CUtensorMap map[N];
    int used = 0, next = 0;
    const CUtensorMap* find(const MapKey& k) const {
        for (int i = 0; i < used; ++i)
            if (key[i] == k) return &map[i];
        return nullptr;
    }
    void put(const MapKey& k, const CUtensorMap& m) {
        const int i = used < N ? used++ : (next = (next + 1) % N);
        key[i] = k;
        map[i] = m;
    }
};
thread_local MapCache t_maps;
thread_local unsigned long long t_map_hits = 0, t_map_misses = 0;

// 2-D row-major tensor (rows x cols, `ld` elements per row) with a (box_cols x box_rows) box,
// 128-byte swizzle (of 16-byte units unless `swizzle` says otherwise), zero fill outside [0, cols) x [0, rows).
int make_map(CUtensorMap* map, bool f16, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
             uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    const MapKey mk = {base, rows, cols, ld, box_cols, box_rows, 0, f16 ? 1 : 0, int(swizzle), 2};
    if (const CUtensorMap* hit = t_maps.find(mk)) { *map = *hit; ++t_map_hits; return 0; }
    ++t_map_misses;
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return DECXB200_EDRIVER;
    const uint64_t esz = f16 ? 2 : 4;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * esz};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) t_maps.put(mk, *map);
    return r == CUDA_SUCCESS ? 0 : DECXB200_EDRIVER;
}

// B (K x N row-major) as a 3-D tensor (column-in-chunk, k, chunk): chunk c holds columns
// [c*chunk_cols, (c+1)*chunk_cols), i.e. dimension 2 has a stride of 128 bytes.  A box of
// (chunk_cols, box_k, box_chunks) then lands in shared memory exactly as box_chunks consecutive
// 2-D boxes would.  A last, partly filled chunk is read at full width, so the caller must make sure
// that ld >= round_up(cols, chunk_cols) (or cols % chunk_cols == 0); what it reads beyond `cols`
// only reaches output columns that are never stored.  Chunks past the last one are zero-filled.
int make_map_b_chunked(CUtensorMap* map, bool f16, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                       uint32_t chunk_cols, uint32_t box_k, uint32_t box_chunks, CUtensorMapSwizzle swizzle) {
    const MapKey mk = {base, rows, cols, ld, chunk_cols, box_k, box_chunks, f16 ? 1 : 0, int(swizzle), 3};
    if (const CUtensorMap* hit = t_maps.find(mk)) { *map = *hit; ++t_map_hits; return 0; }
    ++t_map_misses;
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return DECXB200_EDRIVER;
    const uint64_t esz = f16 ? 2 : 4;
    cuuint64_t dims[3] = {chunk_cols, rows, (cols + chunk_cols - 1) / chunk_cols};
    cuuint64_t strides[2] = {ld * esz, chunk_cols * esz};
    cuuint32_t box[3] = {chunk_cols, box_k, box_chunks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) t_maps.put(mk, *map);
    return r == CUDA_SUCCESS ? 0 : DECXB200_EDRIVER;
}

template <int KIND, int CTAS, int NACC = 1, int FETCH = 0, int BNV = 256>
int launch_gemm(cudaStream_t stream, int dev, const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b0,
                const CUtensorMap& b1, GemmParams p, int max_ctas, const FetchParams* fetch = nullptr, bool pdl = false,
                const CUtensorMap* dmap_given = nullptr) {
    // D through TMA bulk stores (staged in shared memory, 128-byte rows) whenever its rows are 16-byte aligned:
    // that is what makes the stores efficient when D lives in another GPU's memory; DECXB200_TMA_STORE=0 disables
    static const int tma_store_env = [] { const char* e = getenv("DECXB200_TMA_STORE"); return e ? atoi(e) : 1; }();
    CUtensorMap dmap = a0, cmap = a0;
    p.d_tma = 0;
    p.c_tma = 0;
    if (dmap_given != nullptr) {            // the caller built the map of D itself (convolution: a 3-D map)
        dmap = *dmap_given;
        p.d_tma = 1;
    } else if (tma_store_env && p.vec_d) {
        const bool f16 = (KIND == 0);
        if (make_map(&dmap, f16, p.D, p.M, p.N, p.ldd, f16 ? 64 : 32, 32) == 0) p.d_tma = 1;
        // C through the same staging tile (TMA load, same box and swizzle) when its rows are 16-byte aligned too
        static const int tma_c_env = [] { const char* e = getenv("DECXB200_TMA_C"); return e ? atoi(e) : 1; }();
        if (p.d_tma && tma_c_env && p.C != nullptr && p.vec_c &&
            make_map(&cmap, f16, p.C, p.M, p.N, p.ldc, f16 ? 64 : 32, 32) == 0)
            p.c_tma = 1;
    }
    using Cfg = GemmCfg<KIND, CTAS, NACC, FETCH, BNV>;
    auto kern = gemm_tcgen05_kernel<KIND, CTAS, NACC, FETCH, BNV>;
    FetchParams f;
    memset(&f, 0, sizeof(f));
    if (fetch != nullptr) f = *fetch;
    DeviceInfo& di = g_dev[dev];
    {
        std::lock_guard<std::mutex> lk(g_dev_mutex);
        if (di.sm_count == 0) {
            cudaError_t e = cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return int(e);
        }
        if (!di.attr_set[KIND][CTAS - 1][NACC - 1][(FETCH ? 1 : 0) + (BNV == 64 ? 2 : 0) + (BNV == 128 ? 4 : 0)]) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
            if (e != cudaSuccess) return int(e);
            di.attr_set[KIND][CTAS - 1][NACC - 1][(FETCH ? 1 : 0) + (BNV == 64 ? 2 : 0) + (BNV == 128 ? 4 : 0)] = true;
        }
    }
    p.tiles_m = uint32_t((uint64_t(p.M) + Cfg::BM * CTAS - 1) / (Cfg::BM * CTAS));
    p.tiles_n = uint32_t((uint64_t(p.N) + Cfg::BN_TILE - 1) / Cfg::BN_TILE);
    const uint64_t tiles = uint64_t(p.tiles_m) * p.tiles_n;
    if (tiles > 0xFFFFFFFFull) return DECXB200_ETOOLARGE;
    if (p.panel_flags == nullptr) {
        p.n_panels = 1;
        p.panel_end[0] = p.tiles_n;
    } else {
        // the caller gave panel ends in columns: they must fall on tile boundaries (the last one is N)
        for (uint32_t i = 0; i < p.n_panels; ++i) {
            const uint32_t cols = p.panel_end[i];
            if (i + 1 < p.n_panels && (cols % Cfg::BN_TILE) != 0) return DECXB200_EINVAL;
            p.panel_end[i] = (cols + Cfg::BN_TILE - 1) / Cfg::BN_TILE;
        }
        if (p.panel_end[p.n_panels - 1] != p.tiles_n) return DECXB200_EINVAL;
    }
    uint32_t workers = uint32_t(di.sm_count / CTAS);
    if (max_ctas > 0 && uint32_t(max_ctas / CTAS) < workers) workers = uint32_t(max_ctas / CTAS);
    if (workers == 0) workers = 1;
    if (tiles < workers && FETCH == 0) workers = uint32_t(tiles);      // couriers want every SM, tiles or not
    // group height: balance the A rows and B columns the concurrently running tiles touch
    uint32_t g = (CTAS == 1) ? 16 : (NACC == 2 ? 12 : 8);
    if (const char* e = getenv("DECXB200_GROUP_M")) {       // tuning override
        const int v = atoi(e);
        if (v > 0) g = uint32_t(v);
    }
    if (g > p.tiles_m) g = p.tiles_m;
    p.group_m = g;

    // soft lockstep of the persistent CTAs (on unless DECXB200_TILE_SYNC=0); values > 1 set the wait limit in ns
    static const int sync_env = [] { const char* e = getenv("DECXB200_TILE_SYNC"); return e ? atoi(e) : 1; }();
    p.sync_on = (sync_env > 0 && tiles > workers) ? 1u : 0u;
    p.sync_limit_ns = sync_env > 1 ? unsigned(sync_env) : 20000u;
    if (p.sync_on) {
        std::lock_guard<std::mutex> lk(g_dev_mutex);
        p.sync_base = di.ticket_base;
        di.ticket_base += unsigned(tiles);       // every launch adds exactly one ticket per tile
    }

    if constexpr (FETCH > 0) {
        // D forwarding: a ring of two 128 x 512 fp16 tiles per CTA in local memory, mapped like D (64 x 32 boxes)
        const uint64_t ring_rows = uint64_t(workers) * CTAS * 2 * Cfg::BM;
        if (f.fwd_stage != nullptr && NACC == 2 && p.d_tma && f.fwd_stage_bytes >= ring_rows * 1024 &&
            aligned16(f.fwd_stage) && (p.N % 8) == 0 &&
            make_map(&cmap, true, f.fwd_stage, ring_rows, 512, 512, 64, 32) == 0) {
            p.c_tma = 0;
        } else {
            f.fwd_stage = nullptr;
        }
    }

    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(workers * CTAS, 1, 1);
    cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // The kernel just before this one in the stream is the pass that writes the operand planes: let this kernel's
    // CTAs start (barriers, tensor memory) while that pass drains; they wait for it before their first load.
    static const int pdl_env = [] { const char* e = getenv("DECXB200_PDL"); return e ? atoi(e) : 1; }();
    if (pdl && pdl_env != 0 && KIND == 1) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a0, a1, b0, b1, dmap, cmap, p, f);
    if (e != cudaSuccess) return int(e);
    ++t_launches;
    t_variant = KIND * 100 + CTAS * 10 + NACC + (FETCH ? 1000 : 0) + (BNV == 64 ? 5000 : 0) + (BNV == 128 ? 6000 : 0);
    return 0;
}

int default_cta_group() {
    static int v = -1;
    if (v < 0) {
        const char* s = getenv("DECXB200_CTA_GROUP");
        v = (s != nullptr && s[0] == '1') ? 1 : 2;
    }
    return v;
}

}  // namespace

extern "C" {

size_t decxb200_gemm_workspace_bytes(int dtype, uint32_t M, uint32_t N, uint32_t K) {
    if (M == 0 || N == 0 || K == 0) return 0;
    if (dtype == DECXB200_FP32) {
        const uint64_t a = round_up(uint64_t(M) * round_up(K, 32) * 4, 256);
        const uint64_t b = round_up(uint64_t(K) * round_up(N, 32) * 4, 256);
        return size_t(2 * a + 2 * b);
    }
    if (dtype == DECXB200_CPLXF) {
        const uint64_t a = round_up(uint64_t(M) * round_up(2ull * K, 32) * 4, 256);
        const uint64_t b = round_up(2ull * K * round_up(2ull * N, 32) * 4, 256);
        return size_t(2 * a + 2 * b);
    }
    if (dtype == DECXB200_CPLXD) return dxb_host::f64_workspace_bytes(true, M, N, K);
    return 0;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// internal building blocks shared by the device-pointer and the host-pointer entry points
// ------------------------------------------------------------------------------------------
namespace {

struct Scalars {
    float ar = 1.f, ai = 0.f, br = 0.f, bi = 0.f;
};

Scalars read_scalars(int dtype, const void* alpha, const void* beta) {
    Scalars s;
    if (alpha != nullptr) {
        s.ar = static_cast<const float*>(alpha)[0];
        if (dtype == DECXB200_CPLXF) s.ai = static_cast<const float*>(alpha)[1];
    }
    if (beta != nullptr) {
        s.br = static_cast<const float*>(beta)[0];
        if (dtype == DECXB200_CPLXF) s.bi = static_cast<const float*>(beta)[1];
    }
    return s;
}


inline unsigned prepass_blocks(uint64_t work) {
    const uint64_t b = work / 256 + 1;
    return unsigned(b > 148ull * 16 ? 148ull * 16 : b);
}

// tf32 (hi, lo) planes of A.  complex: A is viewed as M x 2K floats with pitch 2*lda.
int prep_a(cudaStream_t stream, bool cplx, const void* A, uint64_t lda, uint32_t M, uint32_t K, float* a_hi,
           float* a_lo, uint64_t ldaw) {
    const uint64_t ldx = cplx ? 2 * lda : lda;
    const uint32_t Kr = cplx ? 2 * K : K;
    const int vec = ((ldx % 4) == 0 && aligned16(A)) ? 1 : 0;
    split_tf32_kernel<<<prepass_blocks(uint64_t(M) * ((Kr + 3) / 4)), 256, 0, stream>>>(
        static_cast<const float*>(A), ldx, M, Kr, a_hi, a_lo, ldaw, vec);
    ++t_launches;
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : int(e);
}

// tf32 planes of both operands of a real product in one launch
int prep_ab(cudaStream_t stream, const void* A, uint64_t lda, const void* B, uint64_t ldb, uint32_t M, uint32_t N, uint32_t K,
            float* a_hi, float* a_lo, uint64_t ldaw, float* b_hi, float* b_lo, uint64_t ldbw) {
    const SplitJob ja{static_cast<const float*>(A), lda, M, K, a_hi, a_lo, ldaw, ((lda % 4) == 0 && aligned16(A)) ? 1 : 0};
    const SplitJob jb{static_cast<const float*>(B), ldb, K, N, b_hi, b_lo, ldbw, ((ldb % 4) == 0 && aligned16(B)) ? 1 : 0};
    const uint64_t work = uint64_t(M) * ((K + 3) / 4) + uint64_t(K) * ((N + 3) / 4);
    split_tf32_pair_kernel<<<prepass_blocks(work), 256, 0, stream>>>(ja, jb);
    ++t_launches;
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : int(e);
}

// tf32 (hi, lo) planes of B (complex: of its 2K x 2N real expansion).
int prep_b(cudaStream_t stream, bool cplx, const void* B, uint64_t ldb, uint32_t K, uint32_t N, float* b_hi,
           float* b_lo, uint64_t ldbw) {
    if (!cplx) {
        const int vec = ((ldb % 4) == 0 && aligned16(B)) ? 1 : 0;
        split_tf32_kernel<<<prepass_blocks(uint64_t(K) * ((N + 3) / 4)), 256, 0, stream>>>(
            static_cast<const float*>(B), ldb, K, N, b_hi, b_lo, ldbw, vec);
    } else {
        expand_split_cplx_b_kernel<<<prepass_blocks(uint64_t(K) * ((N + 1) / 2)), 256, 0, stream>>>(
            static_cast<const float2*>(B), ldb, K, N, b_hi, b_lo, ldbw);
    }
    ++t_launches;
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : int(e);
}

// Timing record of the GEMM kernels for tuning sessions (DECXB200_STATS=1): the kernels add to it, the host reads
// and clears it through decxb200_debug_stats.  Off by default: no kernel touches it then.
__device__ unsigned long long g_debug_stats[32];

void fill_common(GemmParams& p, const Scalars& sc, const void* C, void* D, unsigned* status) {
    memset(&p, 0, sizeof(p));
    p.D = D;
    p.status = status;
    static const int stats_env = [] { const char* e = getenv("DECXB200_STATS"); return e ? atoi(e) : 0; }();
    if (stats_env) {
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_debug_stats) == cudaSuccess) p.stats = static_cast<unsigned long long*>(addr);
    }
    // every wait inside the kernels gives up after this long (DECXB200_WAIT_LIMIT_MS, default 4 s)
    static const unsigned long long limit_ns = [] {
        const char* e = getenv("DECXB200_WAIT_LIMIT_MS");
        const long v = e ? atol(e) : 0;
        return v > 0 ? (unsigned long long)v * 1000000ull : 4000000000ull;
    }();
    p.wait_limit_ns = limit_ns;
    p.alpha_re = sc.ar;
    p.alpha_im = sc.ai;
    p.beta_re = sc.br;
    p.beta_im = sc.bi;
    const bool use_c = (C != nullptr) && (sc.br != 0.f || sc.bi != 0.f);
    p.C = use_c ? C : nullptr;
}

struct PanelGate {            // B arrives in column panels while the kernel runs (see GemmParams)
    uint32_t n = 0;
    uint32_t col_end[MAX_PANELS] = {0};
    const unsigned* flags = nullptr;
    unsigned epoch = 0;
    unsigned long long* stats = nullptr;
};

int run_f16(cudaStream_t stream, int dev, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda,
            const void* B, uint64_t ldb, const void* C, uint64_t ldc, void* D, uint64_t ldd, const Scalars& sc,
            unsigned* status, int cta_group, int max_ctas, const PanelGate* gate = nullptr,
            const FetchParams* fetch = nullptr) {
    if ((lda % 8) != 0 || (ldb % 8) != 0 || !aligned16(A) || !aligned16(B)) return DECXB200_EALIGN;
    GemmParams p;
    fill_common(p, sc, C, D, status);
    p.M = M; p.N = N; p.K = K;
    p.ldd = ldd; p.ldc = ldc;
    p.epi_mode = EPI_REAL;
    p.vec_d = ((ldd % 8) == 0 && aligned16(D)) ? 1 : 0;
    p.vec_c = (p.C != nullptr && (ldc % 8) == 0 && aligned16(C)) ? 1 : 0;
    if (gate != nullptr && gate->n > 0) {
        p.n_panels = gate->n;
        for (uint32_t i = 0; i < gate->n; ++i) p.panel_end[i] = gate->col_end[i];
        p.panel_flags = gate->flags;
        p.panel_epoch = gate->epoch;
        p.stats = gate->stats;
    }
    using C1 = GemmCfg<0, 1>;
    CUtensorMap a0, b0;
    int rc;
    if ((rc = make_map(&a0, true, A, M, K, lda, C1::BK, C1::BM)) != 0) return rc;
    // Two accumulators per tile (256 x 512 per CTA pair) when K is long enough to hide the unoverlapped epilogue
    // and there are at least two rounds of such tiles; DECXB200_NACC=1|2 overrides.
    int nacc = 1;
    const bool force_wide = (cta_group == DECXB200_TILE_256x512);
    if (force_wide) cta_group = 2;
    if (cta_group == 2) {
        static const int nacc_env = [] { const char* e = getenv("DECXB200_NACC"); return e ? atoi(e) : 0; }();
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        // rounds of the persistent grid with either tile; a wide tile is two plain tiles of work at ~8 % less time
        const uint64_t pairs = uint64_t(sms > 0 ? sms : 148) / 2;
        const uint64_t rows256 = (uint64_t(M) + 255) / 256;
        const uint64_t plain = rows256 * ((uint64_t(N) + 255) / 256), wide = rows256 * ((uint64_t(N) + 511) / 512);
        const double t_plain = double((plain + pairs - 1) / pairs);
        const double t_wide = double((wide + pairs - 1) / pairs) * 2.0 * 0.92;
        nacc = (K >= 2048 && t_wide < t_plain) ? 2 : 1;
        if (gate != nullptr && gate->n > 1)                     // panel ends must be tile boundaries
            for (uint32_t i = 0; i + 1 < gate->n; ++i)
                if (gate->col_end[i] % 512 != 0) nacc = 1;
        if (nacc_env == 1 || nacc_env == 2) nacc = nacc_env;
        if (force_wide) {
            nacc = 2;
            if (gate != nullptr && gate->n > 1)
                for (uint32_t i = 0; i + 1 < gate->n; ++i)
                    if (gate->col_end[i] % 512 != 0) return DECXB200_EINVAL;
        }
    }
    // one 3-D load per stage when reading the last column chunk at full width stays inside B's rows
    p.b_chunked_map = ((N % C1::CHUNK_N) == 0 || ldb >= round_up(N, C1::CHUNK_N)) ? 1 : 0;
    if (!p.b_chunked_map) {
        rc = make_map(&b0, true, B, K, N, ldb, C1::CHUNK_N, C1::BK);
    } else if (nacc == 2) {
        rc = make_map_b_chunked(&b0, true, B, K, N, ldb, C1::CHUNK_N, C1::BK, GemmCfg<0, 2, 2>::B_CHUNKS,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    } else if (cta_group == 1) {
        rc = make_map_b_chunked(&b0, true, B, K, N, ldb, C1::CHUNK_N, C1::BK, GemmCfg<0, 1>::B_CHUNKS,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
        rc = make_map_b_chunked(&b0, true, B, K, N, ldb, C1::CHUNK_N, C1::BK, GemmCfg<0, 2>::B_CHUNKS,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (rc != 0) return rc;
    if (fetch != nullptr) {
        if (cta_group != 2) return DECXB200_EINVAL;
        return nacc == 2 ? launch_gemm<0, 2, 2, 2>(stream, dev, a0, a0, b0, b0, p, max_ctas, fetch)
                         : launch_gemm<0, 2, 1, 2>(stream, dev, a0, a0, b0, b0, p, max_ctas, fetch);
    }
    if (nacc == 2) return launch_gemm<0, 2, 2>(stream, dev, a0, a0, b0, b0, p, max_ctas);
    return cta_group == 1 ? launch_gemm<0, 1>(stream, dev, a0, a0, b0, b0, p, max_ctas)
                          : launch_gemm<0, 2>(stream, dev, a0, a0, b0, b0, p, max_ctas);
}

// M x Nr x Kr real 3xTF32 product of pre-split planes (complex: Nr = 2N, Kr = 2K; ldc/ldd in elements)
int run_tf32(cudaStream_t stream, int dev, bool cplx, uint32_t M, uint32_t N, uint32_t K, const float* a_hi,
             const float* a_lo, uint64_t ldaw, const float* b_hi, const float* b_lo, uint64_t ldbw, const void* C,
             uint64_t ldc, void* D, uint64_t ldd, const Scalars& sc, unsigned* status, int cta_group, int max_ctas,
             bool pdl = false) {
    const uint32_t Kr = cplx ? 2 * K : K, Nr = cplx ? 2 * N : N;
    GemmParams p;
    fill_common(p, sc, C, D, status);
    p.M = M; p.N = Nr; p.K = Kr;
    p.ldd = cplx ? 2 * ldd : ldd;
    p.ldc = cplx ? 2 * ldc : ldc;
    p.epi_mode = cplx ? EPI_COMPLEX : EPI_REAL;
    p.vec_d = ((p.ldd % 4) == 0 && aligned16(D)) ? 1 : 0;
    p.vec_c = (p.C != nullptr && (p.ldc % 4) == 0 && aligned16(C)) ? 1 : 0;
    using C1 = GemmCfg<1, 1>;
    CUtensorMap a0, a1, b0, b1;
    int rc;
    if ((rc = make_map(&a0, false, a_hi, M, Kr, ldaw, C1::BK, C1::BM)) != 0) return rc;
    if ((rc = make_map(&a1, false, a_lo, M, Kr, ldaw, C1::BK, C1::BM)) != 0) return rc;
    // the planes are padded to whole 32-float chunks (ldbw), so the one-load-per-stage form is always legal
    p.b_chunked_map = 1;
    // Small problems: 128 x 256 tiles would leave most SMs without one (fp32 1024^3: 32 tiles on 148 SMs), and the
    // call then lasts as long as one SM needs for its tile.  128 x 64 tiles give four times as many.
    static const int narrow_env = [] { const char* e = getenv("DECXB200_NARROW"); return e ? atoi(e) : 1; }();
    const uint64_t tiles_wide = ((uint64_t(M) + 127) / 128) * ((uint64_t(Nr) + 255) / 256);
    const bool narrow = narrow_env != 0 && tiles_wide <= 74;
    if (narrow) cta_group = 1;
    const uint32_t chunks = narrow ? GemmCfg<1, 1, 1, 0, 64>::B_CHUNKS
                                   : (cta_group == 1) ? GemmCfg<1, 1>::B_CHUNKS : GemmCfg<1, 2>::B_CHUNKS;
    if ((rc = make_map_b_chunked(&b0, false, b_hi, Kr, Nr, ldbw, C1::CHUNK_N, C1::BK, chunks,
                                 CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) != 0)
        return rc;
    if ((rc = make_map_b_chunked(&b1, false, b_lo, Kr, Nr, ldbw, C1::CHUNK_N, C1::BK, chunks,
                                 CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) != 0)
        return rc;
    if (narrow) return launch_gemm<1, 1, 1, 0, 64>(stream, dev, a0, a1, b0, b1, p, max_ctas, nullptr, pdl);
    return cta_group == 1 ? launch_gemm<1, 1>(stream, dev, a0, a1, b0, b1, p, max_ctas, nullptr, pdl)
                          : launch_gemm<1, 2>(stream, dev, a0, a1, b0, b1, p, max_ctas, nullptr, pdl);
}

int check_common(int dtype, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda, const void* B,
                 uint64_t ldb, const void* C, uint64_t ldc, const void* D, uint64_t ldd, int& cta_group, int& dev) {
    if (dtype != DECXB200_FP32 && dtype != DECXB200_FP16 && dtype != DECXB200_CPLXF && dtype != DECXB200_FP64 &&
        dtype != DECXB200_CPLXD)
        return DECXB200_EINVAL;
    if (A == nullptr || B == nullptr || D == nullptr) return DECXB200_EINVAL;
    if (M == 0 || N == 0 || K == 0) return DECXB200_EINVAL;
    if (lda < K || ldb < N || ldd < N || (C != nullptr && ldc < N)) return DECXB200_EINVAL;
    if (cta_group == 0) cta_group = default_cta_group();
    if (cta_group != 1 && cta_group != 2 && !(cta_group == DECXB200_TILE_256x512 && dtype == DECXB200_FP16))
        return DECXB200_EINVAL;
    if ((dtype == DECXB200_CPLXF || dtype == DECXB200_CPLXD) &&
        (uint64_t(N) * 2 > 0xFFFFFFFFull || uint64_t(K) * 2 > 0xFFFFFFFFull))
        return DECXB200_ETOOLARGE;
    const cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return int(ce);
    if (dev < 0 || dev >= MAX_DEVICES) return DECXB200_EINVAL;
    return 0;
}

inline uint64_t elem_size(int dtype) {
    switch (dtype) {
        case DECXB200_FP16: return 2;
        case DECXB200_FP32: return 4;
        case DECXB200_CPLXD: return 16;
        default: return 8;                       // fp64, complex fp32
    }
}
inline bool is_f64(int dtype) { return dtype == DECXB200_FP64 || dtype == DECXB200_CPLXD; }
// alpha / beta of the 64-bit types: host pointers to double (double[2] for complex); NULL = 1 / 0
inline void read_scalars_f64(int dtype, const void* alpha, const void* beta, double a[2], double b[2]) {
    a[0] = 1.0; a[1] = 0.0; b[0] = 0.0; b[1] = 0.0;
    if (alpha != nullptr) {
        a[0] = static_cast<const double*>(alpha)[0];
        if (dtype == DECXB200_CPLXD) a[1] = static_cast<const double*>(alpha)[1];
    }
    if (beta != nullptr) {
        b[0] = static_cast<const double*>(beta)[0];
        if (dtype == DECXB200_CPLXD) b[1] = static_cast<const double*>(beta)[1];
    }
}
// device row pitch (elements) of the staging copies: the reference's rule for device matrices, rows
// rounded up to 128 bytes (srcs/modules/core/classes/GPU_Matrix.cu:35-61)
inline uint64_t dev_pitch(int dtype, uint64_t width) { return round_up(width * elem_size(dtype), 128) / elem_size(dtype); }

// streams and events of the host-pointer path, one set per device, created on first use
struct HostPath {
    bool ready = false;
    cudaStream_t h2d = nullptr, comp = nullptr, d2h = nullptr;
    cudaEvent_t ev_b = nullptr, ev_h2d[2] = {nullptr, nullptr}, ev_comp[2] = {nullptr, nullptr},
                ev_d2h[2] = {nullptr, nullptr};
};
HostPath g_host[MAX_DEVICES];

int host_path(int dev, HostPath*& hp) {
    std::lock_guard<std::mutex> lk(g_dev_mutex);
    hp = &g_host[dev];
    if (hp->ready) return 0;
    cudaError_t e;
    if ((e = cudaStreamCreateWithFlags(&hp->h2d, cudaStreamNonBlocking)) != cudaSuccess) return int(e);
    if ((e = cudaStreamCreateWithFlags(&hp->comp, cudaStreamNonBlocking)) != cudaSuccess) return int(e);
    if ((e = cudaStreamCreateWithFlags(&hp->d2h, cudaStreamNonBlocking)) != cudaSuccess) return int(e);
    cudaEvent_t* evs[] = {&hp->ev_b, &hp->ev_h2d[0], &hp->ev_h2d[1], &hp->ev_comp[0], &hp->ev_comp[1],
                          &hp->ev_d2h[0], &hp->ev_d2h[1]};
    for (cudaEvent_t* ev : evs)
        if ((e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming)) != cudaSuccess) return int(e);
    hp->ready = true;
    return 0;
}

// rows of A / D handled per pipeline step of the host-pointer path
uint32_t host_block_rows(uint32_t M) {
    if (M <= 2048) return M;
    // About 32 steps of whole 256-row tiles.  The copies, not the GEMMs, set the pace of this path, and what cannot
    // overlap is the first block's upload and the last block's GEMM + download: small blocks keep both short
    // (fp16 65536 x 16384 x 16384: 8 blocks left 8.5 ms of tail behind the last upload, 32 blocks leave 2 ms).
    uint32_t rb = uint32_t(round_up((uint64_t(M) + 31) / 32, 256));
    if (rb < 1024) rb = 1024;
    return rb > M ? M : rb;
}

struct HostArena {
    uint64_t b_dev, b_hi, b_lo, a_dev[2], a_hi[2], a_lo[2], c_dev[2], d_dev[2], total;
    uint64_t ldb_d, lda_d, ldcd_d, ldaw, ldbw;
    uint32_t rb;
};

HostArena plan_arena(int dtype, uint32_t M, uint32_t N, uint32_t K, bool has_c) {
    HostArena a;
    memset(&a, 0, sizeof(a));
    const uint64_t es = elem_size(dtype);
    const bool cplx = dtype == DECXB200_CPLXF, split = (dtype == DECXB200_FP32 || dtype == DECXB200_CPLXF);
    a.rb = host_block_rows(M);
    a.ldb_d = dev_pitch(dtype, N);
    a.lda_d = dev_pitch(dtype, K);
    a.ldcd_d = dev_pitch(dtype, N);
    a.ldaw = round_up(cplx ? 2ull * K : K, 32);
    a.ldbw = round_up(cplx ? 2ull * N : N, 32);
    uint64_t off = 0;
    auto take = [&](uint64_t bytes) { const uint64_t o = off; off += round_up(bytes, 256); return o; };
    a.b_dev = take(uint64_t(K) * a.ldb_d * es);
    if (split) {
        const uint64_t kb = (cplx ? 2ull * K : K) * a.ldbw * 4;
        a.b_hi = take(kb);
        a.b_lo = take(kb);
    } else if (dtype == DECXB200_CPLXD) {
        a.b_hi = take(dxb_host::f64_workspace_bytes(true, M, N, K));    // real expansion of B
    }
    for (int i = 0; i < 2; ++i) {
        a.a_dev[i] = take(uint64_t(a.rb) * a.lda_d * es);
        if (split) {
            a.a_hi[i] = take(uint64_t(a.rb) * a.ldaw * 4);
            a.a_lo[i] = take(uint64_t(a.rb) * a.ldaw * 4);
        }
        if (has_c) a.c_dev[i] = take(uint64_t(a.rb) * a.ldcd_d * es);
        a.d_dev[i] = take(uint64_t(a.rb) * a.ldcd_d * es);
    }
    a.total = off;
    return a;
}

}  // namespace

int dxb_host::gemm_tf32_planes(cudaStream_t stream, uint32_t M, uint32_t N, uint32_t K, const float* a_hi,
                               const float* a_lo, uint64_t ldaw, const float* b_hi, const float* b_lo, uint64_t ldbw,
                               void* D, uint64_t ldd, unsigned* status) {
    if (a_hi == nullptr || a_lo == nullptr || b_hi == nullptr || b_lo == nullptr || D == nullptr) return DECXB200_EINVAL;
    if (M == 0 || N == 0 || K == 0 || ldaw < K || ldbw < N || ldd < N || (ldaw % 32) != 0 || (ldbw % 32) != 0)
        return DECXB200_EINVAL;
    int dev = 0;
    const cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return int(ce);
    if (dev < 0 || dev >= MAX_DEVICES) return DECXB200_EINVAL;
    return run_tf32(stream, dev, false, M, N, K, a_hi, a_lo, ldaw, b_hi, b_lo, ldbw, nullptr, 0, D, ldd, Scalars(), status,
                    default_cta_group(), 0);
}

// Implicit-GEMM convolution on zero-bordered tf32 planes of the source (see GemmParams::conv_tw).
int dxb_host::conv_tf32_implicit(cudaStream_t stream, const ConvPlanes& c, unsigned* status) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return DECXB200_EDRIVER;
    int dev = 0;
    const cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return int(ce);
    if (dev < 0 || dev >= MAX_DEVICES) return DECXB200_EINVAL;
    if (c.tw != 32 && c.tw != 64 && c.tw != 128) return DECXB200_EINVAL;
    const uint32_t th = 128 / c.tw;
    const uint32_t tiles_x = (c.OW + c.tw - 1) / c.tw, tiles_y = (c.OH + th - 1) / th;
    const uint32_t row_floats = c.kw * c.Cp;                       // contiguous floats of one kernel row at one x
    const uint32_t kbi = (row_floats + 31) / 32;
    CUtensorMap a[2], d;
    for (int pl = 0; pl < 2; ++pl) {
        // (k in kernel row, x, i, y): x advances sx pixels, i one source row, y sy source rows
        cuuint64_t dims[4] = {row_floats, c.OW, c.kh, c.OH};
        cuuint64_t strides[3] = {uint64_t(c.sx) * c.Cp * 4, uint64_t(c.Wp) * c.Cp * 4, uint64_t(c.sy) * c.Wp * c.Cp * 4};
        cuuint32_t box[4] = {32, c.tw, 1, th};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        const CUresult r = enc(&a[pl], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(pl == 0 ? c.src_hi : c.src_lo),
                               dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return DECXB200_EDRIVER;
    }
    {
        cuuint64_t dims[3] = {c.n, c.OW, c.OH};
        cuuint64_t strides[2] = {uint64_t(c.dst_dpitch) * 4, uint64_t(c.dst_wpitch) * c.dst_dpitch * 4};
        cuuint32_t box[3] = {32, 32, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        const CUresult r = enc(&d, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, c.dst, dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return DECXB200_EDRIVER;
    }
    GemmParams p;
    fill_common(p, Scalars(), nullptr, c.dst, status);
    p.M = tiles_x * tiles_y * 128;                                  // every tile row exists; TMA clips at OW / OH
    p.N = c.n;
    p.K = c.kh * kbi * 32;
    p.ldd = c.dst_dpitch;
    p.epi_mode = EPI_REAL;
    p.vec_d = 1;
    p.conv_tw = c.tw;
    p.conv_tiles_x = tiles_x;
    p.conv_kbi = kbi;
    p.b_chunked_map = 1;
    // Tile: up to 64 kernels a single CTA with 64-column accumulators; beyond that CTA pairs (each CTA fetches its own
    // 128 output positions and HALF of the kernel columns -- with hi and lo planes a single CTA could not pull a
    // 128 x 128 tile's operands through its L2 port as fast as it multiplies them) with 128- or 256-column accumulators.
    const int bn = c.n <= 64 ? 64 : (c.n <= 128 ? 128 : 256);
    static const int pair_env = [] { const char* e = getenv("DECXB200_CONV_PAIR"); return e ? atoi(e) : 1; }();
    const bool pair = bn > 64 && pair_env != 0;
    const uint32_t chunks = bn == 64 ? GemmCfg<1, 1, 1, 0, 64>::B_CHUNKS
                            : pair  ? (bn == 128 ? GemmCfg<1, 2, 1, 0, 128>::B_CHUNKS : GemmCfg<1, 2>::B_CHUNKS)
                                    : (bn == 128 ? GemmCfg<1, 1, 1, 0, 128>::B_CHUNKS : GemmCfg<1, 1>::B_CHUNKS);
    using C1 = GemmCfg<1, 1>;
    CUtensorMap b0, b1;
    int rc;
    if ((rc = make_map_b_chunked(&b0, false, c.b_hi, p.K, c.n, c.ldbw, C1::CHUNK_N, C1::BK, chunks,
                                 CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) != 0)
        return rc;
    if ((rc = make_map_b_chunked(&b1, false, c.b_lo, p.K, c.n, c.ldbw, C1::CHUNK_N, C1::BK, chunks,
                                 CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) != 0)
        return rc;
    if (bn == 64) rc = launch_gemm<1, 1, 1, 0, 64>(stream, dev, a[0], a[1], b0, b1, p, 0, nullptr, true, &d);
    else if (pair && bn == 128) rc = launch_gemm<1, 2, 1, 0, 128>(stream, dev, a[0], a[1], b0, b1, p, 0, nullptr, true, &d);
    else if (pair) rc = launch_gemm<1, 2>(stream, dev, a[0], a[1], b0, b1, p, 0, nullptr, true, &d);
    else if (bn == 128) rc = launch_gemm<1, 1, 1, 0, 128>(stream, dev, a[0], a[1], b0, b1, p, 0, nullptr, true, &d);
    else rc = launch_gemm<1, 1>(stream, dev, a[0], a[1], b0, b1, p, 0, nullptr, true, &d);
    if (rc == 0) t_variant += 20000;
    return rc;
}

extern "C" {

int decxb200_gemm_ex(int dtype, void* stream_, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda,
                     const void* B, uint64_t ldb, const void* C, uint64_t ldc, void* D, uint64_t ldd,
                     const void* alpha, const void* beta, void* workspace, size_t workspace_bytes, unsigned* status,
                     int cta_group, int max_ctas) {
    t_launches = 0;
    int dev = 0;
    int rc = check_common(dtype, M, N, K, A, lda, B, ldb, C, ldc, D, ldd, cta_group, dev);
    if (rc != 0) return rc;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (is_f64(dtype)) {
        // no tcgen05 kind for fp64: warp-level DMMA kernel (gemm_f64.cuh); the tile knobs do not apply
        double a[2], b[2];
        read_scalars_f64(dtype, alpha, beta, a, b);
        return dxb_host::run_f64(stream, dtype == DECXB200_CPLXD, M, N, K, A, lda, B, ldb, C, ldc, D, ldd, a, b,
                                 workspace, workspace_bytes);
    }
    const Scalars sc = read_scalars(dtype, alpha, beta);
    if (dtype == DECXB200_FP16)
        return run_f16(stream, dev, M, N, K, A, lda, B, ldb, C, ldc, D, ldd, sc, status, cta_group, max_ctas);

    // fp32 / cplxf: tf32 (hi, lo) planes in the workspace, then one real 3xTF32 GEMM
    const bool cplx = (dtype == DECXB200_CPLXF);
    const uint32_t Kr = cplx ? 2 * K : K, Nr = cplx ? 2 * N : N;
    const size_t need = decxb200_gemm_workspace_bytes(dtype, M, N, K);
    if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return DECXB200_EWORKSPACE;
    const uint64_t ldaw = round_up(Kr, 32), ldbw = round_up(Nr, 32);
    const uint64_t a_bytes = round_up(uint64_t(M) * ldaw * 4, 256);
    const uint64_t b_bytes = round_up(uint64_t(Kr) * ldbw * 4, 256);
    uint8_t* w = static_cast<uint8_t*>(workspace);
    float* a_hi = reinterpret_cast<float*>(w);
    float* a_lo = reinterpret_cast<float*>(w + a_bytes);
    float* b_hi = reinterpret_cast<float*>(w + 2 * a_bytes);
    float* b_lo = reinterpret_cast<float*>(w + 2 * a_bytes + b_bytes);
    if (!cplx) {
        if ((rc = prep_ab(stream, A, lda, B, ldb, M, N, K, a_hi, a_lo, ldaw, b_hi, b_lo, ldbw)) != 0) return rc;
    } else {
        if ((rc = prep_a(stream, cplx, A, lda, M, K, a_hi, a_lo, ldaw)) != 0) return rc;
        if ((rc = prep_b(stream, cplx, B, ldb, K, N, b_hi, b_lo, ldbw)) != 0) return rc;
    }
    return run_tf32(stream, dev, cplx, M, N, K, a_hi, a_lo, ldaw, b_hi, b_lo, ldbw, C, ldc, D, ldd, sc, status,
                    cta_group, max_ctas, true);
}

size_t decxb200_gemm_host_arena_bytes(int dtype, uint32_t M, uint32_t N, uint32_t K, int has_c) {
    if (M == 0 || N == 0 || K == 0) return 0;
    if (dtype != DECXB200_FP32 && dtype != DECXB200_FP16 && dtype != DECXB200_CPLXF && !is_f64(dtype)) return 0;
    return size_t(plan_arena(dtype, M, N, K, has_c != 0).total);
}

int decxb200_gemm_host(int dtype, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda, const void* B,
                       uint64_t ldb, const void* C, uint64_t ldc, void* D, uint64_t ldd, const void* alpha,
                       const void* beta, void* arena, size_t arena_bytes, unsigned* status) {
    t_launches = 0;
    int dev = 0, cta_group = 0;
    int rc = check_common(dtype, M, N, K, A, lda, B, ldb, C, ldc, D, ldd, cta_group, dev);
    if (rc != 0) return rc;
    Scalars sc;
    double a64[2] = {1.0, 0.0}, b64[2] = {0.0, 0.0};
    if (is_f64(dtype)) {
        read_scalars_f64(dtype, alpha, beta, a64, b64);
        sc.br = (b64[0] != 0.0 || b64[1] != 0.0) ? 1.f : 0.f;          // only "is C used" is read from sc below
    } else {
        sc = read_scalars(dtype, alpha, beta);
    }
    const bool use_c = (C != nullptr) && (sc.br != 0.f || sc.bi != 0.f);
    const HostArena ar = plan_arena(dtype, M, N, K, use_c);
    if (arena == nullptr || arena_bytes < ar.total || (reinterpret_cast<uintptr_t>(arena) & 255) != 0)
        return DECXB200_EWORKSPACE;
    HostPath* hp = nullptr;
    if ((rc = host_path(dev, hp)) != 0) return rc;

    const uint64_t es = elem_size(dtype);
    const bool cplx = dtype == DECXB200_CPLXF, split = (dtype == DECXB200_FP32 || dtype == DECXB200_CPLXF);
    uint8_t* base = static_cast<uint8_t*>(arena);
    auto at = [&](uint64_t off) { return base + off; };
    cudaError_t e;
#define DXB_CUDA(call) do { e = (call); if (e != cudaSuccess) { cudaDeviceSynchronize(); return int(e); } } while (0)

    // Large fp16 B: nothing can be computed before B is on the device, and nothing downloaded before something is
    // computed, so a 512 MiB B used to keep the download link idle for its whole upload.  Instead the first row block
    // of A goes up first and B follows in eight column panels; each panel is multiplied with that block as soon as
    // it has arrived and its piece of D goes down while the next panel comes up.
    uint32_t first_rows = 0;
    if (dtype == DECXB200_FP16 && !use_c && N >= 2048 && uint64_t(K) * N * es >= (64ull << 20)) {
        first_rows = M < ar.rb ? M : ar.rb;
        DXB_CUDA(cudaMemcpy2DAsync(at(ar.a_dev[0]), ar.lda_d * es, A, lda * es, uint64_t(K) * es, first_rows,
                                   cudaMemcpyHostToDevice, hp->h2d));
        const uint32_t pw = uint32_t(round_up((uint64_t(N) + 7) / 8, 64));
        for (uint32_t c0 = 0; c0 < N; c0 += pw) {
            const uint32_t w = N - c0 < pw ? N - c0 : pw;
            uint8_t* b_panel = at(ar.b_dev) + uint64_t(c0) * es;
            uint8_t* d_panel = at(ar.d_dev[0]) + uint64_t(c0) * es;
            DXB_CUDA(cudaMemcpy2DAsync(b_panel, ar.ldb_d * es, static_cast<const uint8_t*>(B) + uint64_t(c0) * es, ldb * es,
                                       uint64_t(w) * es, K, cudaMemcpyHostToDevice, hp->h2d));
            DXB_CUDA(cudaEventRecord(hp->ev_b, hp->h2d));
            DXB_CUDA(cudaStreamWaitEvent(hp->comp, hp->ev_b, 0));
            rc = run_f16(hp->comp, dev, first_rows, w, K, at(ar.a_dev[0]), ar.lda_d, b_panel, ar.ldb_d, nullptr, 0, d_panel,
                         ar.ldcd_d, sc, status, cta_group, 0);
            if (rc != 0) { cudaDeviceSynchronize(); return rc; }
            DXB_CUDA(cudaEventRecord(hp->ev_comp[0], hp->comp));
            DXB_CUDA(cudaStreamWaitEvent(hp->d2h, hp->ev_comp[0], 0));
            DXB_CUDA(cudaMemcpy2DAsync(static_cast<uint8_t*>(D) + uint64_t(c0) * es, ldd * es, d_panel, ar.ldcd_d * es,
                                       uint64_t(w) * es, first_rows, cudaMemcpyDeviceToHost, hp->d2h));
        }
        DXB_CUDA(cudaEventRecord(hp->ev_d2h[0], hp->d2h));
    } else {
        // B: one copy, one split; every row block of A reuses it
        DXB_CUDA(cudaMemcpy2DAsync(at(ar.b_dev), ar.ldb_d * es, B, ldb * es, uint64_t(N) * es, K, cudaMemcpyHostToDevice,
                                   hp->h2d));
        DXB_CUDA(cudaEventRecord(hp->ev_b, hp->h2d));
        DXB_CUDA(cudaStreamWaitEvent(hp->comp, hp->ev_b, 0));
    }
    if (split) {
        rc = prep_b(hp->comp, cplx, at(ar.b_dev), ar.ldb_d, K, N, reinterpret_cast<float*>(at(ar.b_hi)),
                    reinterpret_cast<float*>(at(ar.b_lo)), ar.ldbw);
        if (rc != 0) { cudaDeviceSynchronize(); return rc; }
    }
    // row blocks: H2D of block i+1 and D2H of block i-1 overlap the GEMM of block i
    uint32_t step = first_rows ? 1 : 0;                     // buffers 0 are in use by the first block's panels
    for (uint32_t r0 = first_rows; r0 < M; r0 += ar.rb, ++step) {
        const uint32_t rows = (M - r0 < ar.rb) ? M - r0 : ar.rb;
        const int b = int(step & 1u);
        const uint8_t* a_src = static_cast<const uint8_t*>(A) + uint64_t(r0) * lda * es;
        if (step >= 2) DXB_CUDA(cudaStreamWaitEvent(hp->h2d, hp->ev_comp[b], 0));   // staging buffers free again
        DXB_CUDA(cudaMemcpy2DAsync(at(ar.a_dev[b]), ar.lda_d * es, a_src, lda * es, uint64_t(K) * es, rows,
                                   cudaMemcpyHostToDevice, hp->h2d));
        if (use_c) {
            const uint8_t* c_src = static_cast<const uint8_t*>(C) + uint64_t(r0) * ldc * es;
            DXB_CUDA(cudaMemcpy2DAsync(at(ar.c_dev[b]), ar.ldcd_d * es, c_src, ldc * es, uint64_t(N) * es, rows,
                                       cudaMemcpyHostToDevice, hp->h2d));
        }
        DXB_CUDA(cudaEventRecord(hp->ev_h2d[b], hp->h2d));
        DXB_CUDA(cudaStreamWaitEvent(hp->comp, hp->ev_h2d[b], 0));
        if (step >= 2) DXB_CUDA(cudaStreamWaitEvent(hp->comp, hp->ev_d2h[b], 0));  // D staging buffer drained
        const void* c_dev = use_c ? at(ar.c_dev[b]) : nullptr;
        if (is_f64(dtype)) {
            const size_t wsb = dxb_host::f64_workspace_bytes(dtype == DECXB200_CPLXD, M, N, K);
            rc = dxb_host::run_f64(hp->comp, dtype == DECXB200_CPLXD, rows, N, K, at(ar.a_dev[b]), ar.lda_d,
                                   at(ar.b_dev), ar.ldb_d, c_dev, ar.ldcd_d, at(ar.d_dev[b]), ar.ldcd_d, a64, b64,
                                   wsb ? at(ar.b_hi) : nullptr, wsb, step > 0);
        } else if (!split) {
            rc = run_f16(hp->comp, dev, rows, N, K, at(ar.a_dev[b]), ar.lda_d, at(ar.b_dev), ar.ldb_d, c_dev,
                         ar.ldcd_d, at(ar.d_dev[b]), ar.ldcd_d, sc, status, cta_group, 0);
        } else {
            float* a_hi = reinterpret_cast<float*>(at(ar.a_hi[b]));
            float* a_lo = reinterpret_cast<float*>(at(ar.a_lo[b]));
            rc = prep_a(hp->comp, cplx, at(ar.a_dev[b]), ar.lda_d, rows, K, a_hi, a_lo, ar.ldaw);
            if (rc == 0)
                rc = run_tf32(hp->comp, dev, cplx, rows, N, K, a_hi, a_lo, ar.ldaw,
                              reinterpret_cast<float*>(at(ar.b_hi)), reinterpret_cast<float*>(at(ar.b_lo)), ar.ldbw,
                              c_dev, ar.ldcd_d, at(ar.d_dev[b]), ar.ldcd_d, sc, status, cta_group, 0, true);
        }
        if (rc != 0) { cudaDeviceSynchronize(); return rc; }
        DXB_CUDA(cudaEventRecord(hp->ev_comp[b], hp->comp));
        DXB_CUDA(cudaStreamWaitEvent(hp->d2h, hp->ev_comp[b], 0));
        uint8_t* d_dst = static_cast<uint8_t*>(D) + uint64_t(r0) * ldd * es;
        DXB_CUDA(cudaMemcpy2DAsync(d_dst, ldd * es, at(ar.d_dev[b]), ar.ldcd_d * es, uint64_t(N) * es, rows,
                                   cudaMemcpyDeviceToHost, hp->d2h));
        DXB_CUDA(cudaEventRecord(hp->ev_d2h[b], hp->d2h));
    }
    DXB_CUDA(cudaStreamSynchronize(hp->d2h));
    DXB_CUDA(cudaStreamSynchronize(hp->comp));
    DXB_CUDA(cudaStreamSynchronize(hp->h2d));
#undef DXB_CUDA
    if (status != nullptr) {
        unsigned st = 0;
        e = cudaMemcpy(&st, status, sizeof(st), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return int(e);
        if (st != 0) return DECXB200_EKERNEL;
    }
    return 0;
}

int decxb200_gemm(int dtype, void* stream, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda,
                  const void* B, uint64_t ldb, const void* C, uint64_t ldc, void* D, uint64_t ldd, const void* alpha,
                  const void* beta, void* workspace, size_t workspace_bytes, unsigned* status) {
    return decxb200_gemm_ex(dtype, stream, M, N, K, A, lda, B, ldb, C, ldc, D, ldd, alpha, beta, workspace,
                            workspace_bytes, status, 0, 0);
}

// ------------------------------------------------------------------------------------------
// fp32 GEMM whose scratch is a fixed array inside the library (see the header for who needs it)
// ------------------------------------------------------------------------------------------
// Lives in every context that loads this module until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[DECXB200_NOALLOC_SCRATCH_BYTES];

namespace {
// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address, so the
// address each device gave the array is looked up once per device and kept here.
void* g_noalloc_addr[MAX_DEVICES] = {nullptr};

int noalloc_scratch_address(int dev, void** out) {
    std::lock_guard<std::mutex> lk(g_dev_mutex);
    if (g_noalloc_addr[dev] == nullptr) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);   // for the CURRENT device (= dev)
        if (e != cudaSuccess) return int(e);
        if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255) != 0) return DECXB200_EWORKSPACE;
        g_noalloc_addr[dev] = ptr;
    }
    *out = g_noalloc_addr[dev];
    return 0;
}
}  // namespace

int decxb200_gemm_fp32_noalloc(void* stream_, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda,
                               const void* B, uint64_t ldb, const void* C, uint64_t ldc, void* D, uint64_t ldd,
                               const void* alpha, const void* beta, unsigned* status) {
    t_launches = 0;
    int dev = 0, cta_group = 0;
    int rc = check_common(DECXB200_FP32, M, N, K, A, lda, B, ldb, C, ldc, D, ldd, cta_group, dev);
    if (rc != 0) return rc;
    const size_t need = decxb200_gemm_workspace_bytes(DECXB200_FP32, M, N, K);
    if (need > size_t(DECXB200_NOALLOC_SCRATCH_BYTES)) return DECXB200_ETOOLARGE;
    void* scratch = nullptr;
    if ((rc = noalloc_scratch_address(dev, &scratch)) != 0) return rc;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    // The array still holds the planes of whichever call used it last.  The one-load-per-stage form of
    // the B tensor map reads the padding columns of the B planes, which the split pass does not write:
    // clear the part this call uses so that nothing stale (for instance NaN bit patterns) is ever read.
    const cudaError_t ce = cudaMemsetAsync(scratch, 0, need, stream);
    if (ce != cudaSuccess) return int(ce);
    const Scalars sc = read_scalars(DECXB200_FP32, alpha, beta);
    const uint64_t ldaw = round_up(K, 32), ldbw = round_up(N, 32);
    const uint64_t a_bytes = round_up(uint64_t(M) * ldaw * 4, 256);
    const uint64_t b_bytes = round_up(uint64_t(K) * ldbw * 4, 256);
    uint8_t* w = static_cast<uint8_t*>(scratch);
    float* a_hi = reinterpret_cast<float*>(w);
    float* a_lo = reinterpret_cast<float*>(w + a_bytes);
    float* b_hi = reinterpret_cast<float*>(w + 2 * a_bytes);
    float* b_lo = reinterpret_cast<float*>(w + 2 * a_bytes + b_bytes);
    if ((rc = prep_a(stream, false, A, lda, M, K, a_hi, a_lo, ldaw)) != 0) return rc;
    if ((rc = prep_b(stream, false, B, ldb, K, N, b_hi, b_lo, ldbw)) != 0) return rc;
    return run_tf32(stream, dev, false, M, N, K, a_hi, a_lo, ldaw, b_hi, b_lo, ldbw, C, ldc, D, ldd, sc, status,
                    cta_group, 0);
}

int decxb200_gemm_fp16_panels(void* stream_, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda,
                              const void* B, uint64_t ldb, void* D, uint64_t ldd, unsigned* status, uint32_t n_panels,
                              const uint32_t* panel_col_end, const unsigned* panel_flags, unsigned epoch,
                              int max_ctas, int tile) {
    t_launches = 0;
    int dev = 0, cta_group = (tile == DECXB200_TILE_256x512) ? tile : 2;
    int rc = check_common(DECXB200_FP16, M, N, K, A, lda, B, ldb, nullptr, 0, D, ldd, cta_group, dev);
    if (rc != 0) return rc;
    if (n_panels == 0 || n_panels > uint32_t(MAX_PANELS) || panel_col_end == nullptr || panel_flags == nullptr)
        return DECXB200_EINVAL;
    PanelGate g;
    g.n = n_panels;
    uint32_t prev = 0;
    for (uint32_t i = 0; i < n_panels; ++i) {
        if (panel_col_end[i] <= prev || panel_col_end[i] > N) return DECXB200_EINVAL;
        g.col_end[i] = prev = panel_col_end[i];
    }
    if (prev != N) return DECXB200_EINVAL;
    g.flags = panel_flags;
    g.epoch = epoch;
    return run_f16(reinterpret_cast<cudaStream_t>(stream_), dev, M, N, K, A, lda, B, ldb, nullptr, 0, D, ldd, Scalars(),
                   status, cta_group, max_ctas, &g);
}

// scratch layout: [0, 256) batch counters, [256, 512) timing record (32 x u64), [512, ...) job table
constexpr size_t FETCH_TABLE_OFF = 512;
// ... then one counter per job (push jobs count their batches there)
size_t decxb200_fetch_scratch_bytes(uint32_t n_jobs) {
    return FETCH_TABLE_OFF + size_t(round_up(uint64_t(n_jobs) * sizeof(FetchJob), 256)) + size_t(round_up(uint64_t(n_jobs) * 4, 256));
}

size_t decxb200_fetch_d_stage_bytes(void) { return size_t(256) * 2 * 128 * 1024; }     // up to 256 CTAs

int decxb200_gemm_fp16_fetch(void* stream_, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda, void* B,
                             uint64_t ldb, void* D, uint64_t ldd, unsigned* status, uint32_t n_panels,
                             const uint32_t* panel_col_end, unsigned* ready_flags, unsigned* pub_flags, unsigned epoch,
                             const decxb200_fetch_job* jobs, uint32_t n_jobs, void* scratch, size_t scratch_bytes,
                             int max_ctas, int tile) {
    return decxb200_gemm_fp16_fetch_staged(stream_, M, N, K, A, lda, B, ldb, D, ldd, status, n_panels, panel_col_end,
                                           ready_flags, pub_flags, epoch, jobs, n_jobs, scratch, scratch_bytes, max_ctas,
                                           tile, nullptr, 0);
}

int decxb200_gemm_fp16_fetch_staged(void* stream_, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda, void* B,
                                    uint64_t ldb, void* D, uint64_t ldd, unsigned* status, uint32_t n_panels,
                                    const uint32_t* panel_col_end, unsigned* ready_flags, unsigned* pub_flags,
                                    unsigned epoch, const decxb200_fetch_job* jobs, uint32_t n_jobs, void* scratch,
                                    size_t scratch_bytes, int max_ctas, int tile, void* d_stage, size_t d_stage_bytes) {
    t_launches = 0;
    int dev = 0, cta_group = (tile == DECXB200_TILE_256x512) ? tile : 2;
    int rc = check_common(DECXB200_FP16, M, N, K, A, lda, B, ldb, nullptr, 0, D, ldd, cta_group, dev);
    if (rc != 0) return rc;
    if (n_panels == 0 || n_panels > uint32_t(MAX_PANELS) || panel_col_end == nullptr) return DECXB200_EINVAL;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    PanelGate g;
    g.n = n_panels;
    uint32_t prev = 0;
    for (uint32_t i = 0; i < n_panels; ++i) {
        if (panel_col_end[i] <= prev || panel_col_end[i] > N) return DECXB200_EINVAL;
        g.col_end[i] = prev = panel_col_end[i];
    }
    if (prev != N) return DECXB200_EINVAL;
    g.flags = ready_flags;
    g.epoch = epoch;
    if (n_jobs == 0) {
        // nothing to bring in (this GPU already holds all of B): the plain or the flag-gated GEMM
        return run_f16(stream, dev, M, N, K, A, lda, B, ldb, nullptr, 0, D, ldd, Scalars(), status, cta_group, max_ctas,
                       ready_flags != nullptr ? &g : nullptr);
    }
    bool any_pull = false;
    if (jobs != nullptr)
        for (uint32_t i = 0; i < n_jobs; ++i) any_pull = any_pull || jobs[i].dst == nullptr;
    // a GPU that only pushes (the owner) needs no flags of its own: its tiles read the B it already holds
    if (jobs == nullptr || (any_pull && (ready_flags == nullptr || pub_flags == nullptr)) || scratch == nullptr ||
        scratch_bytes < decxb200_fetch_scratch_bytes(n_jobs) || (reinterpret_cast<uintptr_t>(scratch) & 255) != 0)
        return DECXB200_EWORKSPACE;
    FetchParams f;
    memset(&f, 0, sizeof(f));
    std::vector<FetchJob> table(n_jobs);
    for (uint32_t i = 0; i < n_jobs; ++i) {
        const decxb200_fetch_job& j = jobs[i];
        if (j.panel >= n_panels || (j.col0 % 8) != 0 || (j.cols % 8) != 0 || j.cols == 0) return DECXB200_EINVAL;
        const uint32_t lo = j.panel ? g.col_end[j.panel - 1] : 0u;
        if (j.col0 < lo || uint64_t(j.col0) + j.cols > g.col_end[j.panel]) return DECXB200_EINVAL;
        if (uint64_t(j.row0) + j.rows > K) return DECXB200_EINVAL;
        if (j.rows != 0 && (j.src == nullptr || !aligned16(j.src))) return DECXB200_EINVAL;
        if (j.rows == 0 && j.gate == nullptr) return DECXB200_EINVAL;     // a piece nobody delivers and nobody flags
        if (j.dst != nullptr && (j.rows == 0 || !aligned16(j.dst) || (j.publish != 0 && j.publish != DECXB200_FETCH_MULTICAST)))
            return DECXB200_EINVAL;
        if (j.dst == nullptr && j.publish > 1) return DECXB200_EINVAL;
        if (j.publish == DECXB200_FETCH_MULTICAST && j.notify == nullptr) return DECXB200_EINVAL;
        if (j.dst == nullptr && j.notify != nullptr) return DECXB200_EINVAL;
        FetchJob& t = table[i];
        t.src = static_cast<const uint8_t*>(j.src);
        t.gate = j.gate;
        t.dst = static_cast<uint8_t*>(j.dst);
        t.notify = j.notify;
        t.row0 = j.row0; t.rows = j.rows;
        t.byte0 = j.col0 * 2; t.bytes = j.cols * 2;
        t.panel = j.panel;
        t.publish = j.dst != nullptr ? j.publish : (j.publish ? 1u : 0u);
        const uint32_t nb = fetch_job_batches(t.rows, t.bytes);
        if (t.dst == nullptr) {
            f.need[t.panel] += nb;
            if (t.publish) f.pub_need[t.panel] += nb;
        }
        f.total_batches += nb;
    }
    if (any_pull)
        for (uint32_t i = 0; i < n_panels; ++i)
            if (f.need[i] == 0) return DECXB200_EINVAL;   // a panel nothing delivers would never be flagged
    uint8_t* sc = static_cast<uint8_t*>(scratch);
    cudaError_t e;
    const size_t table_bytes = size_t(round_up(uint64_t(n_jobs) * sizeof(FetchJob), 256));
    if ((e = cudaMemsetAsync(sc, 0, FETCH_TABLE_OFF, stream)) != cudaSuccess) return int(e);
    if ((e = cudaMemsetAsync(sc + FETCH_TABLE_OFF + table_bytes, 0, size_t(n_jobs) * 4, stream)) != cudaSuccess) return int(e);
    // pageable source: staged by the runtime before the call returns, so `table` may go out of scope
    if ((e = cudaMemcpyAsync(sc + FETCH_TABLE_OFF, table.data(), size_t(n_jobs) * sizeof(FetchJob), cudaMemcpyHostToDevice,
                             stream)) != cudaSuccess)
        return int(e);
    f.jobs = reinterpret_cast<const FetchJob*>(sc + FETCH_TABLE_OFF);
    g.stats = reinterpret_cast<unsigned long long*>(sc + 256);
    f.n_jobs = n_jobs;
    f.dst = static_cast<uint8_t*>(B);
    f.pitch = ldb * 2;
    f.arrived = reinterpret_cast<unsigned*>(sc);
    f.published = reinterpret_cast<unsigned*>(sc + 64);
    f.next_batch = reinterpret_cast<unsigned*>(sc + 128);
    f.job_done = reinterpret_cast<unsigned*>(sc + FETCH_TABLE_OFF + table_bytes);
    f.ready_flags = ready_flags;
    f.pub_flags = pub_flags;
    f.epoch = epoch;
    f.fwd_stage = static_cast<uint8_t*>(d_stage);
    f.fwd_stage_bytes = d_stage_bytes;
    return run_f16(stream, dev, M, N, K, A, lda, B, ldb, nullptr, 0, D, ldd, Scalars(), status, cta_group, max_ctas,
                   any_pull ? &g : nullptr, &f);
}

int decxb200_copy2d_async(void* stream, void* dst, size_t dpitch, const void* src, size_t spitch, size_t width_bytes,
                          size_t rows) {
    const cudaError_t e = cudaMemcpy2DAsync(dst, dpitch, src, spitch, width_bytes, rows, cudaMemcpyDefault,
                                            reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : int(e);
}

int decxb200_write_flag_async(void* stream, unsigned* flag, unsigned value) {
    typedef CUresult (*WriteValueFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    static WriteValueFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<WriteValueFn>(p);
    });
    if (fn == nullptr || flag == nullptr) return DECXB200_EDRIVER;
    const CUresult r = fn(reinterpret_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(flag), value, 0);
    return r == CUDA_SUCCESS ? 0 : DECXB200_EDRIVER;
}

int decxb200_ipc_alloc(size_t bytes, void** dptr) {
    if (dptr == nullptr || bytes == 0) return DECXB200_EINVAL;
    const cudaError_t e = cudaMalloc(dptr, bytes);   // a whole allocation: IPC handles name allocations
    return e == cudaSuccess ? 0 : int(e);
}

int decxb200_ipc_free(void* dptr) {
    const cudaError_t e = cudaFree(dptr);
    return e == cudaSuccess ? 0 : int(e);
}

int decxb200_ipc_export(void* dptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (dptr == nullptr || handle == nullptr) return DECXB200_EINVAL;
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, dptr);
    if (e != cudaSuccess) return int(e);
    memcpy(handle, &h, 64);
    return 0;
}

int decxb200_ipc_open(const unsigned char handle[64], void** peer_ptr) {
    if (handle == nullptr || peer_ptr == nullptr) return DECXB200_EINVAL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    const cudaError_t e = cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess);
    return e == cudaSuccess ? 0 : int(e);
}

int decxb200_ipc_close(void* peer_ptr) {
    const cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
    return e == cudaSuccess ? 0 : int(e);
}

int decxb200_last_launch_count(void) { return t_launches; }
int decxb200_last_kernel_variant(void) { return t_variant; }
int decxb200_debug_stats(unsigned long long out[32]) {
    if (out == nullptr) return DECXB200_EINVAL;
    cudaError_t e = cudaMemcpyFromSymbol(out, g_debug_stats, sizeof(unsigned long long) * 32);   // waits for earlier kernels
    if (e != cudaSuccess) return int(e);
    static const unsigned long long zeros[32] = {0};
    e = cudaMemcpyToSymbol(g_debug_stats, zeros, sizeof(zeros));
    return e == cudaSuccess ? 0 : int(e);
}
void decxb200_tensor_map_cache_stats(unsigned long long* hits, unsigned long long* misses) {
    if (hits != nullptr) *hits = t_map_hits;
    if (misses != nullptr) *misses = t_map_misses;
}

const char* decxb200_strerror(int code) {
    switch (code) {
        case 0: return "success";
        case DECXB200_EINVAL: return "invalid argument (null pointer, zero extent, pitch smaller than width, unknown dtype)";
        case DECXB200_EALIGN: return "fp16 operands need 16-byte aligned base addresses and pitches that are multiples of 8 elements";
        case DECXB200_EWORKSPACE: return "workspace is missing, not 256-byte aligned, or smaller than decxb200_gemm_workspace_bytes()";
        case DECXB200_EDRIVER: return "cuTensorMapEncodeTiled is unavailable or rejected the tensor (no CUDA driver / no sm_100 device?)";
        case DECXB200_ETOOLARGE: return "problem extent beyond what this entry point supports";
        case DECXB200_EKERNEL: return "a bounded wait inside the GEMM kernel expired";
        default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error";
    }
}

const char* decxb200_version(void) { return "0.1"; }

}  // extern "C"
