// extern "C" layer, second part: matrix-vector products, transpose, element casts and the fp64 GEMMs.
// See include/decx_b200.h for the contracts.
#include <cstring>
#include <mutex>

#include "../../include/decx_b200.h"
#include "capi_shared.h"
#include "gemm_f64.cuh"
#include "conv2d.cuh"
#include "gemv.cuh"
#include "transpose_cast.cuh"

using namespace dxb;
using dxb_host::aligned16;
using dxb_host::round_up;

namespace {

inline int last_error() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : int(e);
}

// ------------------------------------------------------------------------------------------------ GEMV planning
struct GemvPlan {
    uint32_t slices, slice_len, out_len, red_len;
    size_t part_bytes;        // bytes of one partial element
};

// trans == 0: y[rows] = A x (reduce over the cols); trans == 1: y[cols] = x A (reduce over the rows)
GemvPlan plan_gemv(int dtype, int accu, int trans, uint32_t rows, uint32_t cols) {
    GemvPlan g;
    const uint32_t vec = (dtype == DECXB200_FP16) ? 8 : 4;
    g.out_len = trans ? cols : rows;
    g.red_len = trans ? rows : cols;
    g.part_bytes = (dtype == DECXB200_FP16 && accu == DECXB200_FP16_ACCU_L3) ? 2 : 4;
    uint32_t want = 1;
    if (!trans) {
        // one warp per row and slice: aim at >= 32 warps per SM of a 148-SM part
        if (rows < 4736) want = (4736 + rows - 1) / rows;
        const uint32_t unit = 32 * vec * GEMV_UNROLL;                  // elements one warp iteration covers
        const uint32_t max_slices = (cols + unit - 1) / unit;
        if (want > max_slices) want = max_slices;
        if (want < 1) want = 1;
        g.slice_len = uint32_t(round_up((uint64_t(cols) + want - 1) / want, unit));
    } else {
        const uint32_t col_blocks = (cols + 32 * vec - 1) / (32 * vec);
        if (col_blocks < 1776) want = (1776 + col_blocks - 1) / col_blocks;      // about 12 CTAs per SM
        const uint32_t unit = GEMV_WARPS * GEMV_UNROLL * 4;            // rows: a few unrolled rounds per warp
        const uint32_t max_slices = (rows + unit - 1) / unit;
        if (want > max_slices) want = max_slices;
        if (want < 1) want = 1;
        g.slice_len = uint32_t(round_up((uint64_t(rows) + want - 1) / want, GEMV_WARPS * GEMV_UNROLL));
    }
    g.slices = (g.red_len + g.slice_len - 1) / g.slice_len;
    if (g.slices > 65535) {                                            // gridDim.y limit
        g.slices = 65535;
        g.slice_len = uint32_t(round_up((uint64_t(g.red_len) + 65534) / 65535, 32 * vec * GEMV_UNROLL));
        g.slices = (g.red_len + g.slice_len - 1) / g.slice_len;
    }
    return g;
}

template <typename T, typename ACC, typename OUT>
int launch_gemv(cudaStream_t s, int trans, const GemvPlan& g, uint32_t rows, uint32_t cols, const void* A, uint64_t lda,
                const void* x, void* y, void* ws) {
    const bool vec_ok = aligned16(A) && (lda * sizeof(T)) % 16 == 0 && (trans || aligned16(x));
    void* out = g.slices == 1 ? y : ws;
    if (!trans) {
        dim3 grid((rows + GEMV_WARPS - 1) / GEMV_WARPS, g.slices);
        gemv_rows_kernel<T, ACC, OUT><<<grid, GEMV_WARPS * 32, 0, s>>>(static_cast<const T*>(A), lda,
                                                                        static_cast<const T*>(x), out, rows, cols,
                                                                        g.slice_len, vec_ok ? 1 : 0);
    } else {
        constexpr uint32_t V = 16 / sizeof(T);
        dim3 grid((cols + 32 * V - 1) / (32 * V), g.slices);
        gemv_cols_kernel<T, ACC, OUT><<<grid, GEMV_WARPS * 32, 0, s>>>(static_cast<const T*>(A), lda,
                                                                        static_cast<const T*>(x), out, rows, cols,
                                                                        g.slice_len, vec_ok ? 1 : 0);
    }
    dxb_host::count_launch();
    int rc = last_error();
    if (rc != 0 || g.slices == 1) return rc;
    gemv_finish_kernel<ACC, OUT><<<(g.out_len + 255) / 256, 256, 0, s>>>(
        static_cast<const typename ACC::part_t*>(ws), g.slices, g.out_len, static_cast<OUT*>(y));
    dxb_host::count_launch();
    return last_error();
}

}  // namespace

extern "C" {

size_t decxb200_gemv_workspace_bytes(int dtype, int fp16_accu, int trans, uint32_t rows, uint32_t cols) {
    if (rows == 0 || cols == 0 || (dtype != DECXB200_FP32 && dtype != DECXB200_FP16)) return 0;
    const GemvPlan g = plan_gemv(dtype, fp16_accu, trans, rows, cols);
    return g.slices > 1 ? size_t(round_up(uint64_t(g.slices) * g.out_len * g.part_bytes, 256)) : 0;
}

int decxb200_gemv(int dtype, int fp16_accu, int trans, void* stream_, uint32_t rows, uint32_t cols, const void* A,
                  uint64_t lda, const void* x, void* y, void* workspace, size_t workspace_bytes) {
    dxb_host::reset_launches();
    if (dtype != DECXB200_FP32 && dtype != DECXB200_FP16) return DECXB200_EINVAL;
    if (A == nullptr || x == nullptr || y == nullptr || rows == 0 || cols == 0 || lda < cols) return DECXB200_EINVAL;
    if (dtype == DECXB200_FP16 && (fp16_accu < DECXB200_FP16_ACCU_L1 || fp16_accu > DECXB200_FP16_ACCU_L3))
        return DECXB200_EINVAL;
    GemvPlan g = plan_gemv(dtype, fp16_accu, trans, rows, cols);
    if (g.slices > 1) {
        const size_t need = size_t(g.slices) * g.out_len * g.part_bytes;
        if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15) != 0) {
            g.slices = 1;                 // no scratch: one slice does the whole reduction (slower on skinny shapes)
            g.slice_len = g.red_len;
        }
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
    if (dtype == DECXB200_FP32) return launch_gemv<float, AccF32, float>(s, trans, g, rows, cols, A, lda, x, y, workspace);
    if (fp16_accu == DECXB200_FP16_ACCU_L1)
        return launch_gemv<__half, AccF32, float>(s, trans, g, rows, cols, A, lda, x, y, workspace);
    if (fp16_accu == DECXB200_FP16_ACCU_L2)
        return launch_gemv<__half, AccF32, __half>(s, trans, g, rows, cols, A, lda, x, y, workspace);
    return launch_gemv<__half, AccF16, __half>(s, trans, g, rows, cols, A, lda, x, y, workspace);
}

int decxb200_transpose(int elem_bytes, void* stream_, uint32_t rows, uint32_t cols, const void* src, uint64_t lds,
                       void* dst, uint64_t ldd) {
    dxb_host::reset_launches();
    if (src == nullptr || dst == nullptr || rows == 0 || cols == 0 || lds < cols || ldd < rows) return DECXB200_EINVAL;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
    const uintptr_t sa = reinterpret_cast<uintptr_t>(src), da = reinterpret_cast<uintptr_t>(dst);
    auto grid = [&](uint32_t tile) { return dim3((cols + tile - 1) / tile, (rows + tile - 1) / tile); };
    switch (elem_bytes) {
        case 1:
            transpose_scalar_kernel<uint8_t><<<grid(32), 256, 0, s>>>(static_cast<const uint8_t*>(src), lds,
                                                                      static_cast<uint8_t*>(dst), ldd, rows, cols);
            break;
        case 2:
            if ((lds % 8) == 0 && (ldd % 8) == 0 && (sa % 16) == 0 && (da % 16) == 0)
                transpose_b2_vec_kernel<<<dim3((cols + 127) / 128, (rows + 63) / 64), 256, 0, s>>>(
                    static_cast<const uint16_t*>(src), lds, static_cast<uint16_t*>(dst), ldd, rows, cols);
            else
                transpose_scalar_kernel<uint16_t><<<grid(32), 256, 0, s>>>(static_cast<const uint16_t*>(src), lds,
                                                                           static_cast<uint16_t*>(dst), ldd, rows, cols);
            break;
        case 4:
            if ((lds % 4) == 0 && (ldd % 4) == 0 && (sa % 16) == 0 && (da % 16) == 0)
                transpose_b4_vec_kernel<<<grid(64), 256, 0, s>>>(static_cast<const uint32_t*>(src), lds,
                                                                 static_cast<uint32_t*>(dst), ldd, rows, cols);
            else
                transpose_words_kernel<uint32_t, 32><<<grid(32), 256, 0, s>>>(static_cast<const uint32_t*>(src), lds,
                                                                              static_cast<uint32_t*>(dst), ldd, rows, cols);
            break;
        case 8:
            transpose_words_kernel<uint64_t, 32><<<grid(32), 256, 0, s>>>(static_cast<const uint64_t*>(src), lds,
                                                                          static_cast<uint64_t*>(dst), ldd, rows, cols);
            break;
        case 16:
            if ((sa % 16) != 0 || (da % 16) != 0) return DECXB200_EALIGN;
            transpose_words_kernel<uint4, 16><<<grid(16), 256, 0, s>>>(static_cast<const uint4*>(src), lds,
                                                                       static_cast<uint4*>(dst), ldd, rows, cols);
            break;
        default: return DECXB200_EINVAL;
    }
    dxb_host::count_launch();
    return last_error();
}

int decxb200_cast2d(int kind, void* stream_, uint32_t rows, uint32_t cols, const void* src, uint64_t lds, void* dst,
                    uint64_t ldd) {
    dxb_host::reset_launches();
    if (src == nullptr || dst == nullptr || rows == 0 || cols == 0 || lds < cols || ldd < cols) return DECXB200_EINVAL;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
    const uint64_t work = uint64_t(rows) * ((cols + 1) / 2);
    // a thread converts four groups per round: a quarter of the blocks, capped at 32 per SM
    const unsigned blocks = unsigned(work / 1024 + 1 > 148ull * 32 ? 148ull * 32 : work / 1024 + 1);
#define DXB_CAST(KIND)                                                                                              \
    {                                                                                                               \
        using S = CastTypes<KIND>::S;                                                                               \
        using D = CastTypes<KIND>::D;                                                                               \
        const int vec = aligned16(src) && aligned16(dst) && (lds * sizeof(S)) % 16 == 0 && (ldd * sizeof(D)) % 16 == 0; \
        cast2d_kernel<KIND><<<blocks, 256, 0, s>>>(static_cast<const S*>(src), lds, static_cast<D*>(dst), ldd, rows,  \
                                                   cols, vec);                                                      \
    }                                                                                                               \
    break;
    switch (kind) {
        case DECXB200_CAST_F32_F16: DXB_CAST(CAST_F32_F16)
        case DECXB200_CAST_F16_F32: DXB_CAST(CAST_F16_F32)
        case DECXB200_CAST_F32_F64: DXB_CAST(CAST_F32_F64)
        case DECXB200_CAST_F64_F32: DXB_CAST(CAST_F64_F32)
        case DECXB200_CAST_I32_F32: DXB_CAST(CAST_I32_F32)
        case DECXB200_CAST_F32_I32: DXB_CAST(CAST_F32_I32)
        default: return DECXB200_EINVAL;
    }
#undef DXB_CAST
    dxb_host::count_launch();
    return last_error();
}

// ------------------------------------------------------------------------------------------------ conv2d
static int conv2d_geometry(uint32_t H, uint32_t W, uint32_t C, uint32_t kh, uint32_t kw, uint32_t sx, uint32_t sy, int extend,
                           uint32_t dst_wpitch, Conv2dGeom& g) {
    if (H == 0 || W == 0 || C == 0 || kh == 0 || kw == 0 || sx == 0 || sy == 0) return DECXB200_EINVAL;
    memset(&g, 0, sizeof(g));
    g.H = H; g.W = W; g.C = C; g.kh = kh; g.kw = kw; g.sx = sx; g.sy = sy;
    if (extend == DECXB200_EXTEND_NONE) {
        if (kh > H || kw > W) return DECXB200_EINVAL;
        g.OH = (H - kh + 1) / sy;
        g.OW = (W - kw + 1) / sx;
        g.Hlim = H;
    } else if (extend == DECXB200_EXTEND_CONSTANT) {
        g.OH = H / sy;
        g.OW = W / sx;
        g.py = kh / 2;
        g.px = kw / 2;
        g.Hlim = g.OH * sy;
    } else {
        return DECXB200_EINVAL;
    }
    if (g.OH == 0 || g.OW == 0) return DECXB200_EINVAL;
    g.dst_wpitch = dst_wpitch ? dst_wpitch : g.OW;
    if (g.dst_wpitch < g.OW) return DECXB200_EINVAL;
    g.Cp = (C + 3) / 4 * 4;
    const uint64_t kc = uint64_t(kh) * kw * g.Cp, rows = uint64_t(g.OH) * g.dst_wpitch;
    if (kc > 0xFFFFFFFFull || rows > 0xFFFFFFFFull) return DECXB200_ETOOLARGE;
    g.Kc = uint32_t(kc);
    return 0;
}

int decxb200_conv2d_fp32_out_dims(uint32_t H, uint32_t W, uint32_t kh, uint32_t kw, uint32_t sx, uint32_t sy, int extend,
                                  uint32_t* OH, uint32_t* OW) {
    Conv2dGeom g;
    const int rc = conv2d_geometry(H, W, 1, kh, kw, sx, sy, extend, 0, g);
    if (rc != 0) return rc;
    if (OH) *OH = g.OH;
    if (OW) *OW = g.OW;
    return 0;
}

namespace {
// which form a convolution takes, and what each needs
struct ConvPlan {
    bool implicit;
    uint32_t tw, Hp, Wp, kbi;
    uint64_t M, ldaw, ldbw, Kb;            // materialised: rows of the im2col matrix, its pitch; both: B's pitch and rows
    uint64_t a_bytes, b_bytes;             // per plane
};
ConvPlan conv_plan(const Conv2dGeom& g, uint32_t n_kernels, uint32_t dst_dpitch) {
    static const int implicit_env = [] { const char* e = getenv("DECXB200_CONV_IMPLICIT"); return e ? atoi(e) : 1; }();
    ConvPlan p;
    memset(&p, 0, sizeof(p));
    p.ldbw = round_up(n_kernels, 32);
    p.implicit = implicit_env != 0 && (n_kernels % 4) == 0 && (dst_dpitch % 4) == 0;
    if (p.implicit) {
        // tile row width: least padding of the output columns, wider on ties
        uint64_t best = ~0ull;
        for (uint32_t tw : {128u, 64u, 32u}) {
            const uint32_t th = 128 / tw;
            const uint64_t cover = uint64_t((g.OW + tw - 1) / tw) * tw * ((g.OH + th - 1) / th) * th;
            if (cover < best) { best = cover; p.tw = tw; }
        }
        p.Hp = (g.OH - 1) * g.sy + g.kh;
        p.Wp = (g.OW - 1) * g.sx + g.kw;
        p.kbi = (g.kw * g.Cp + 31) / 32;
        p.Kb = uint64_t(g.kh) * p.kbi * 32;
        p.a_bytes = round_up(uint64_t(p.Hp) * p.Wp * g.Cp * 4, 256);
    } else {
        p.M = uint64_t(g.OH) * g.dst_wpitch;
        p.ldaw = round_up(g.Kc, 32);
        p.Kb = g.Kc;
        p.a_bytes = round_up(p.M * p.ldaw * 4, 256);
    }
    p.b_bytes = round_up(p.Kb * p.ldbw * 4, 256);
    return p;
}
}  // namespace

size_t decxb200_conv2d_fp32_workspace_bytes(uint32_t H, uint32_t W, uint32_t C, uint32_t kh, uint32_t kw, uint32_t n_kernels,
                                            uint32_t sx, uint32_t sy, int extend, uint32_t dst_wpitch, uint32_t dst_dpitch) {
    Conv2dGeom g;
    if (n_kernels == 0 || conv2d_geometry(H, W, C, kh, kw, sx, sy, extend, dst_wpitch, g) != 0) return 0;
    const ConvPlan p = conv_plan(g, n_kernels, dst_dpitch ? dst_dpitch : n_kernels);
    return size_t(2 * p.a_bytes + 2 * p.b_bytes);
}

int decxb200_conv2d_fp32(void* stream_, const void* src, uint32_t H, uint32_t W, uint32_t C, uint32_t src_wpitch,
                         uint32_t src_dpitch, const void* kernels, uint32_t kh, uint32_t kw, uint32_t n_kernels,
                         uint32_t kernel_wpitch, uint32_t kernel_dpitch, uint64_t kernel_stride, void* dst,
                         uint32_t dst_wpitch, uint32_t dst_dpitch, uint32_t sx, uint32_t sy, int extend, void* workspace,
                         size_t workspace_bytes, unsigned* status) {
    dxb_host::reset_launches();
    Conv2dGeom g;
    if (src == nullptr || kernels == nullptr || dst == nullptr || n_kernels == 0) return DECXB200_EINVAL;
    int rc = conv2d_geometry(H, W, C, kh, kw, sx, sy, extend, dst_wpitch, g);
    if (rc != 0) return rc;
    if (src_wpitch < W || src_dpitch < C || kernel_wpitch < kw || kernel_dpitch < C || dst_dpitch < n_kernels)
        return DECXB200_EINVAL;
    g.src_wpitch = src_wpitch;
    g.src_dpitch = src_dpitch;
    // a destination that is not 16-byte aligned takes the materialised form whatever its pitch
    const ConvPlan p = conv_plan(g, n_kernels, aligned16(dst) ? dst_dpitch : 1);
    const size_t need = size_t(2 * p.a_bytes + 2 * p.b_bytes);
    if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return DECXB200_EWORKSPACE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
    uint8_t* w = static_cast<uint8_t*>(workspace);
    float* a_hi = reinterpret_cast<float*>(w);
    float* a_lo = reinterpret_cast<float*>(w + p.a_bytes);
    float* b_hi = reinterpret_cast<float*>(w + 2 * p.a_bytes);
    float* b_lo = reinterpret_cast<float*>(w + 2 * p.a_bytes + p.b_bytes);
    const int vec = aligned16(src) && (src_dpitch % 4) == 0;
    auto blocks = [](uint64_t work) { return unsigned(work / 256 + 1 > 148ull * 32 ? 148ull * 32 : work / 256 + 1); };
    const uint32_t row_pad = p.implicit ? p.kbi * 32 : g.kw * g.Cp;
    pack_kernels_split_kernel<<<blocks(p.Kb * ((n_kernels + 3) / 4)), 256, 0, s>>>(
        static_cast<const float*>(kernels), kernel_stride, kernel_wpitch, kernel_dpitch, kh, kw, C, g.Cp, n_kernels, row_pad,
        b_hi, b_lo, p.ldbw);
    if (p.implicit) {
        pad_split_src_kernel<<<blocks(uint64_t(p.Hp) * p.Wp * (g.Cp / 4)), 256, 0, s>>>(static_cast<const float*>(src), a_hi,
                                                                                        a_lo, p.Hp, p.Wp, g, vec);
        if ((rc = last_error()) != 0) return rc;
        dxb_host::ConvPlanes c;
        memset(&c, 0, sizeof(c));
        c.src_hi = a_hi; c.src_lo = a_lo; c.Wp = p.Wp; c.Cp = g.Cp;
        c.b_hi = b_hi; c.b_lo = b_lo; c.ldbw = p.ldbw;
        c.kh = kh; c.kw = kw; c.n = n_kernels; c.sx = sx; c.sy = sy; c.OH = g.OH; c.OW = g.OW;
        c.dst = static_cast<float*>(dst); c.dst_wpitch = g.dst_wpitch; c.dst_dpitch = dst_dpitch;
        c.tw = p.tw;
        rc = dxb_host::conv_tf32_implicit(s, c, status);
    } else {
        im2col_split_kernel<<<blocks(p.M * g.kh * g.kw * (g.Cp / 4)), 256, 0, s>>>(static_cast<const float*>(src), a_hi, a_lo,
                                                                                    p.ldaw, g, vec);
        if ((rc = last_error()) != 0) return rc;
        rc = dxb_host::gemm_tf32_planes(s, uint32_t(p.M), n_kernels, g.Kc, a_hi, a_lo, p.ldaw, b_hi, b_lo, p.ldbw, dst,
                                        dst_dpitch, status);
    }
    dxb_host::count_launch(2);
    return rc;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------ fp64 GEMM
namespace dxb_host {

size_t f64_workspace_bytes(bool cplx, uint32_t M, uint32_t N, uint32_t K) {
    (void)M;
    if (!cplx) return 0;
    return size_t(round_up(2ull * K * (2ull * N) * 8, 256));
}

int run_f64(cudaStream_t stream, bool cplx, uint32_t M, uint32_t N, uint32_t K, const void* A, uint64_t lda,
            const void* B, uint64_t ldb, const void* C, uint64_t ldc, void* D, uint64_t ldd, const double alpha[2],
            const double beta[2], void* workspace, size_t workspace_bytes, bool b_expanded) {
    static std::mutex mtx;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return int(e);
    {
        std::lock_guard<std::mutex> lk(mtx);
        if (dev >= 0 && dev < 64 && !attr_set[dev]) {
            e = cudaFuncSetAttribute(gemm_f64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F64_SMEM_BYTES);
            if (e != cudaSuccess) return int(e);
            attr_set[dev] = true;
        }
    }
    GemmF64Params p;
    memset(&p, 0, sizeof(p));
    p.alpha_re = alpha[0]; p.alpha_im = cplx ? alpha[1] : 0.0;
    p.beta_re = beta[0]; p.beta_im = cplx ? beta[1] : 0.0;
    const bool use_c = C != nullptr && (p.beta_re != 0.0 || p.beta_im != 0.0);
    p.C = use_c ? static_cast<const double*>(C) : nullptr;
    p.D = static_cast<double*>(D);
    p.A = static_cast<const double*>(A);
    p.complex_epilogue = cplx ? 1 : 0;
    if (!cplx) {
        p.B = static_cast<const double*>(B);
        p.M = M; p.N = N; p.K = K;
        p.lda = lda; p.ldb = ldb; p.ldc = ldc; p.ldd = ldd;
    } else {
        const size_t need = f64_workspace_bytes(true, M, N, K);
        if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
            return DECXB200_EWORKSPACE;
        const uint64_t ldw = 2ull * N;
        const uint64_t total = uint64_t(K) * N;
        const unsigned blocks = unsigned(total / 256 + 1 > 148ull * 16 ? 148ull * 16 : total / 256 + 1);
        if (!b_expanded) {
            expand_cplxd_b_kernel<<<blocks, 256, 0, stream>>>(static_cast<const double2*>(B), ldb, K, N,
                                                              static_cast<double*>(workspace), ldw);
            count_launch();
            if ((e = cudaGetLastError()) != cudaSuccess) return int(e);
        }
        p.B = static_cast<const double*>(workspace);
        p.M = M; p.N = 2 * N; p.K = 2 * K;
        p.lda = 2 * lda; p.ldb = ldw; p.ldc = 2 * ldc; p.ldd = 2 * ldd;
    }
    p.vec_a = (aligned16(p.A) && (p.lda % 2) == 0) ? 1 : 0;
    p.vec_b = (aligned16(p.B) && (p.ldb % 2) == 0) ? 1 : 0;
    const uint32_t tiles_m = (p.M + F64_BM - 1) / F64_BM;
    p.tiles_n = (p.N + F64_BN - 1) / F64_BN;
    p.group_m = tiles_m < 8 ? tiles_m : 8;
    const uint64_t tiles = uint64_t(tiles_m) * p.tiles_n;
    if (tiles > 0x7FFFFFFFull) return DECXB200_ETOOLARGE;
    gemm_f64_kernel<<<unsigned(tiles), F64_THREADS, F64_SMEM_BYTES, stream>>>(p);
    count_launch();
    e = cudaGetLastError();
    return e == cudaSuccess ? 0 : int(e);
}

}  // namespace dxb_host
