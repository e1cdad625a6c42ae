// extern "C" layer of the B200 GEMM path: argument checks, tensor-map encoding,
// workspace carving, pre-pass and GEMM launches.  See include/decx_b200.h.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/decx_b200.h"
#include "gemm_sm100.cuh"
#include "prepass.cuh"

namespace {

using namespace dxb;

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
    int sm_count = 0;
    bool attr_set[2][2] = {{false, false}, {false, false}};
    int max_pairs[2] = {0, 0};
};
DeviceInfo g_dev[MAX_DEVICES];
std::mutex g_dev_mutex;

thread_local int t_launches = 0;

inline uint64_t round_up(uint64_t x, uint64_t m) { return (x + m - 1) / m * m; }

// 2-D row-major tensor (rows x cols, `ld` elements per row) with a (box_cols x box_rows) box,
// 128-byte swizzle (of 16-byte units unless `swizzle` says otherwise), zero fill outside [0, cols) x [0, rows).
int make_map(CUtensorMap* map, bool f16, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
             uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
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
    return r == CUDA_SUCCESS ? 0 : DECXB200_EDRIVER;
}

template <int KIND, int CTAS>
int launch_gemm(cudaStream_t stream, int dev, const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b0,
                const CUtensorMap& b1, GemmParams p, int max_ctas) {
    using Cfg = GemmCfg<KIND, CTAS>;
    auto kern = gemm_tcgen05_kernel<KIND, CTAS>;
    DeviceInfo& di = g_dev[dev];
    {
        std::lock_guard<std::mutex> lk(g_dev_mutex);
        if (di.sm_count == 0) {
            cudaError_t e = cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return int(e);
        }
        if (!di.attr_set[KIND][CTAS - 1]) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
            if (e != cudaSuccess) return int(e);
            di.attr_set[KIND][CTAS - 1] = true;
        }
    }
    p.tiles_m = uint32_t((uint64_t(p.M) + Cfg::BM * CTAS - 1) / (Cfg::BM * CTAS));
    p.tiles_n = uint32_t((uint64_t(p.N) + Cfg::BN - 1) / Cfg::BN);
    const uint64_t tiles = uint64_t(p.tiles_m) * p.tiles_n;
    if (tiles > 0xFFFFFFFFull) return DECXB200_ETOOLARGE;
    uint32_t workers = uint32_t(di.sm_count / CTAS);
    if (max_ctas > 0 && uint32_t(max_ctas / CTAS) < workers) workers = uint32_t(max_ctas / CTAS);
    if (workers == 0) workers = 1;
    if (tiles < workers) workers = uint32_t(tiles);
    // group height: balance the A rows and B columns the concurrently running tiles touch
    uint32_t g = (CTAS == 1) ? 16 : 8;
    if (g > p.tiles_m) g = p.tiles_m;
    p.group_m = g;

    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(workers * CTAS, 1, 1);
    cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a0, a1, b0, b1, p);
    if (e != cudaSuccess) return int(e);
    ++t_launches;
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
    return 0;
}

int decxb200_gemm_ex(int dtype, void* stream_, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda,
                     const void* B, uint64_t ldb, const void* C, uint64_t ldc, void* D, uint64_t ldd,
                     const void* alpha, const void* beta, void* workspace, size_t workspace_bytes, unsigned* status,
                     int cta_group, int max_ctas) {
    t_launches = 0;
    if (dtype != DECXB200_FP32 && dtype != DECXB200_FP16 && dtype != DECXB200_CPLXF) return DECXB200_EINVAL;
    if (A == nullptr || B == nullptr || D == nullptr) return DECXB200_EINVAL;
    if (M == 0 || N == 0 || K == 0) return DECXB200_EINVAL;
    if (lda < K || ldb < N || ldd < N || (C != nullptr && ldc < N)) return DECXB200_EINVAL;
    if (cta_group == 0) cta_group = default_cta_group();
    if (cta_group != 1 && cta_group != 2) return DECXB200_EINVAL;
    if (dtype == DECXB200_CPLXF && (uint64_t(N) * 2 > 0xFFFFFFFFull || uint64_t(K) * 2 > 0xFFFFFFFFull))
        return DECXB200_ETOOLARGE;

    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return int(ce);
    if (dev < 0 || dev >= MAX_DEVICES) return DECXB200_EINVAL;

    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.D = D;
    p.status = status;
    p.wait_limit_ns = 4000000000ull;
    p.alpha_re = 1.f;
    p.alpha_im = 0.f;
    p.beta_re = 0.f;
    p.beta_im = 0.f;
    if (alpha != nullptr) {
        p.alpha_re = static_cast<const float*>(alpha)[0];
        if (dtype == DECXB200_CPLXF) p.alpha_im = static_cast<const float*>(alpha)[1];
    }
    if (beta != nullptr) {
        p.beta_re = static_cast<const float*>(beta)[0];
        if (dtype == DECXB200_CPLXF) p.beta_im = static_cast<const float*>(beta)[1];
    }
    const bool use_c = (C != nullptr) && (p.beta_re != 0.f || p.beta_im != 0.f);
    p.C = use_c ? C : nullptr;

    CUtensorMap a0, a1, b0, b1;
    int rc;
    if (dtype == DECXB200_FP16) {
        if ((lda % 8) != 0 || (ldb % 8) != 0 || (reinterpret_cast<uintptr_t>(A) & 15) != 0 ||
            (reinterpret_cast<uintptr_t>(B) & 15) != 0)
            return DECXB200_EALIGN;
        p.M = M; p.N = N; p.K = K;
        p.ldd = ldd; p.ldc = ldc;
        p.epi_mode = EPI_REAL;
        p.vec_d = ((ldd % 8) == 0 && (reinterpret_cast<uintptr_t>(D) & 15) == 0) ? 1 : 0;
        p.vec_c = (use_c && (ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
        using C1 = GemmCfg<0, 1>;
        if ((rc = make_map(&a0, true, A, M, K, lda, C1::BK, C1::BM)) != 0) return rc;
        if ((rc = make_map(&b0, true, B, K, N, ldb, C1::CHUNK_N, C1::BK)) != 0) return rc;
        a1 = a0;
        b1 = b0;
        return cta_group == 1 ? launch_gemm<0, 1>(stream, dev, a0, a1, b0, b1, p, max_ctas)
                              : launch_gemm<0, 2>(stream, dev, a0, a1, b0, b1, p, max_ctas);
    }

    // fp32 / cplxf: tf32 (hi, lo) planes in the workspace, then one real 3xTF32 GEMM
    const bool cplx = (dtype == DECXB200_CPLXF);
    const uint32_t Kr = cplx ? 2 * K : K;      // real extents seen by the MMA
    const uint32_t Nr = cplx ? 2 * N : N;
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

    {
        // A (complex: viewed as M x 2K floats with pitch 2*lda)
        const uint64_t ldx = cplx ? 2 * lda : lda;
        const int vec = ((ldx % 4) == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0) ? 1 : 0;
        const uint64_t work = uint64_t(M) * ((Kr + 3) / 4);
        const unsigned blocks = unsigned(work / 256 + 1 > 148ull * 16 ? 148ull * 16 : work / 256 + 1);
        split_tf32_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float*>(A), ldx, M, Kr, a_hi, a_lo, ldaw, vec);
        ++t_launches;
    }
    if (!cplx) {
        const int vec = ((ldb % 4) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0) ? 1 : 0;
        const uint64_t work = uint64_t(K) * ((N + 3) / 4);
        const unsigned blocks = unsigned(work / 256 + 1 > 148ull * 16 ? 148ull * 16 : work / 256 + 1);
        split_tf32_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float*>(B), ldb, K, N, b_hi, b_lo, ldbw, vec);
        ++t_launches;
    } else {
        const uint64_t work = uint64_t(K) * ((N + 1) / 2);
        const unsigned blocks = unsigned(work / 256 + 1 > 148ull * 16 ? 148ull * 16 : work / 256 + 1);
        expand_split_cplx_b_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float2*>(B), ldb, K, N, b_hi, b_lo,
                                                               ldbw);
        ++t_launches;
    }
    ce = cudaGetLastError();
    if (ce != cudaSuccess) return int(ce);

    p.M = M; p.N = Nr; p.K = Kr;
    p.ldd = cplx ? 2 * ldd : ldd;
    p.ldc = cplx ? 2 * ldc : ldc;
    p.epi_mode = cplx ? EPI_COMPLEX : EPI_REAL;
    p.vec_d = ((p.ldd % 4) == 0 && (reinterpret_cast<uintptr_t>(D) & 15) == 0) ? 1 : 0;
    p.vec_c = (use_c && (p.ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
    using C1 = GemmCfg<1, 1>;
    if ((rc = make_map(&a0, false, a_hi, M, Kr, ldaw, C1::BK, C1::BM)) != 0) return rc;
    if ((rc = make_map(&a1, false, a_lo, M, Kr, ldaw, C1::BK, C1::BM)) != 0) return rc;
    if ((rc = make_map(&b0, false, b_hi, Kr, Nr, ldbw, C1::CHUNK_N, C1::BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) != 0) return rc;
    if ((rc = make_map(&b1, false, b_lo, Kr, Nr, ldbw, C1::CHUNK_N, C1::BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) != 0) return rc;
    return cta_group == 1 ? launch_gemm<1, 1>(stream, dev, a0, a1, b0, b1, p, max_ctas)
                          : launch_gemm<1, 2>(stream, dev, a0, a1, b0, b1, p, max_ctas);
}

int decxb200_gemm(int dtype, void* stream, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda,
                  const void* B, uint64_t ldb, const void* C, uint64_t ldc, void* D, uint64_t ldd, const void* alpha,
                  const void* beta, void* workspace, size_t workspace_bytes, unsigned* status) {
    return decxb200_gemm_ex(dtype, stream, M, N, K, A, lda, B, ldb, C, ldc, D, ldd, alpha, beta, workspace,
                            workspace_bytes, status, 0, 0);
}

int decxb200_last_launch_count(void) { return t_launches; }

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
