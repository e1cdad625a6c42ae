// GPU test of the C++ drop-in, written the way a DECX user program is written (compare the reference's
// samples/Matrix_Multiplication/MatMul.cpp): InitCuda, Create*MatrixRef(type, width, height), fill through
// ptr<T>(row, col), de::Memcpy, de::blas::cuda::GEMM, de::Memcpy back, look at de::GetLastError().
// Results are checked against an fp64 triple loop (fp32 for fp16) with the path's metric
//   max |D - Dref| / (|A row| * |B column|)  <=  1e-5 (fp32, complex)   1e-2 (fp16).
#include <cmath>
#include <complex>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "DECX.h"

static int g_fail = 0;
#define CHECK(c) do { if (!(c)) { std::printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #c); ++g_fail; } } while (0)

static uint32_t g_seed = 1;
static float rnd() {   // U[-1, 1)
    g_seed = g_seed * 1664525u + 1013904223u;
    return float(int32_t(g_seed >> 8) - (1 << 23)) / float(1 << 23);
}

template <typename T> struct Ops;
template <> struct Ops<float> {
    static constexpr de::_DATA_TYPES_FLAGS_ type = de::_FP32_;
    typedef double wide;
    static float make() { return rnd(); }
    static wide up(float x) { return x; }
    static double mag(wide x) { return std::fabs(x); }
    static de::Number num(double re, double) { return de::Number(float(re)); }
    static wide scal(double re, double) { return re; }
    static constexpr double tol = 1e-5;
};
template <> struct Ops<de::CPf> {
    static constexpr de::_DATA_TYPES_FLAGS_ type = de::_COMPLEX_F32_;
    typedef std::complex<double> wide;
    static de::CPf make() { return de::CPf(rnd(), rnd()); }
    static wide up(de::CPf x) { return wide(x.real, x.image); }
    static double mag(wide x) { return std::abs(x); }
    static de::Number num(double re, double im) { return de::Number(de::CPf(float(re), float(im))); }
    static wide scal(double re, double im) { return wide(re, im); }
    static constexpr double tol = 1e-5;
};
template <> struct Ops<de::Half> {
    static constexpr de::_DATA_TYPES_FLAGS_ type = de::_FP16_;
    typedef double wide;
    static de::Half make() { return de::Float2Half(rnd() * 0.5f); }
    static wide up(de::Half x) { return de::Half2Float(x); }
    static double mag(wide x) { return std::fabs(x); }
    static de::Number num(double re, double) { return de::Number(de::Float2Half(float(re))); }
    static wide scal(double re, double) { return re; }
    static constexpr double tol = 1e-2;
};

template <> struct Ops<double> {
    static constexpr de::_DATA_TYPES_FLAGS_ type = de::_FP64_;
    typedef long double wide;
    static double make() { return double(rnd()) + double(rnd()) * 0x1p-24; }
    static wide up(double x) { return x; }
    static double mag(wide x) { return double(fabsl(x)); }
    static de::Number num(double re, double) { return de::Number(re); }
    static wide scal(double re, double) { return re; }
    static constexpr double tol = 1e-13;
};
template <> struct Ops<de::CPd> {
    static constexpr de::_DATA_TYPES_FLAGS_ type = de::_COMPLEX_F64_;
    typedef std::complex<long double> wide;
    static de::CPd make() { return de::CPd(double(rnd()) + double(rnd()) * 0x1p-24, double(rnd())); }
    static wide up(de::CPd x) { return wide(x.real, x.image); }
    static double mag(wide x) { return double(std::abs(x)); }
    static de::Number num(double re, double im) { return de::Number(de::CPd(re, im)); }
    static wide scal(double re, double im) { return wide(re, im); }
    static constexpr double tol = 1e-13;
};

// M x N x K problem through the device-matrix overloads (fused when `fused`), and through the host-matrix ones
template <typename T>
static void run_case(uint32_t M, uint32_t N, uint32_t K, bool fused, bool host_overload) {
    typedef Ops<T> O;
    typedef typename O::wide W;
    de::Matrix& A = de::CreateMatrixRef(O::type, K, M);
    de::Matrix& B = de::CreateMatrixRef(O::type, N, K);
    de::Matrix& C = de::CreateMatrixRef(O::type, N, M);
    de::Matrix& D = de::CreateMatrixRef(O::type, N, M);
    for (uint32_t i = 0; i < M; ++i) for (uint32_t k = 0; k < K; ++k) *A.ptr<T>(i, k) = O::make();
    for (uint32_t k = 0; k < K; ++k) for (uint32_t j = 0; j < N; ++j) *B.ptr<T>(k, j) = O::make();
    for (uint32_t i = 0; i < M; ++i) for (uint32_t j = 0; j < N; ++j) *C.ptr<T>(i, j) = O::make();
    const double ar = host_overload ? 1.0 : 0.75, ai = host_overload ? 0.0 : -0.5;
    const double br = host_overload ? 1.0 : -1.25, bi = host_overload ? 0.0 : 0.5;
    const bool cplx = (O::type == de::_COMPLEX_F32_ || O::type == de::_COMPLEX_F64_);
    de::ResetLastError();
    if (host_overload) {
        if (fused) de::blas::cuda::GEMM(A, B, C, D); else de::blas::cuda::GEMM(A, B, D);
    } else {
        de::GPU_Matrix& dA = de::CreateGPUMatrixRef(O::type, K, M);
        de::GPU_Matrix& dB = de::CreateGPUMatrixRef(O::type, N, K);
        de::GPU_Matrix& dC = de::CreateGPUMatrixRef(O::type, N, M);
        de::GPU_Matrix& dD = de::CreateGPUMatrixRef();                    // shaped by GEMM
        de::Memcpy(A, dA, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(K, M), de::DECX_MEMCPY_H2D);
        de::Memcpy(B, dB, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(N, K), de::DECX_MEMCPY_H2D);
        de::Memcpy(C, dC, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(N, M), de::DECX_MEMCPY_H2D);
        if (fused) de::blas::cuda::GEMM(dA, dB, dC, dD, O::num(ar, cplx ? ai : 0), O::num(br, cplx ? bi : 0));
        else de::blas::cuda::GEMM(dA, dB, dD);
        CHECK(dD.Width() == N && dD.Height() == M && dD.Type() == O::type);
        de::Memcpy(D, dD, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(N, M), de::DECX_MEMCPY_D2H);
        dA.release(); dB.release(); dC.release(); dD.release();
    }
    CHECK(de::GetLastError()->error_type == de::DECX_SUCCESS);
    if (de::GetLastError()->error_type != de::DECX_SUCCESS) std::printf("  DH: %s\n", de::GetLastError()->error_string);
    std::vector<double> rn(M, 0.0), cn(N, 0.0);
    for (uint32_t i = 0; i < M; ++i) { for (uint32_t k = 0; k < K; ++k) rn[i] += std::norm(O::up(*A.ptr<T>(i, k))); rn[i] = std::sqrt(rn[i]); }
    for (uint32_t j = 0; j < N; ++j) { for (uint32_t k = 0; k < K; ++k) cn[j] += std::norm(O::up(*B.ptr<T>(k, j))); cn[j] = std::sqrt(cn[j]); }
    const W alpha = fused ? O::scal(ar, cplx ? ai : 0) : O::scal(1, 0), beta = fused ? O::scal(br, cplx ? bi : 0) : O::scal(0, 0);
    double worst = 0.0;
    for (uint32_t i = 0; i < M; ++i)
        for (uint32_t j = 0; j < N; ++j) {
            W acc = O::scal(0, 0);
            for (uint32_t k = 0; k < K; ++k) acc += O::up(*A.ptr<T>(i, k)) * O::up(*B.ptr<T>(k, j));
            const W ref = alpha * acc + beta * O::up(*C.ptr<T>(i, j));
            const double m = O::mag(O::up(*D.ptr<T>(i, j)) - ref) / (rn[i] * cn[j]);
            if (!(m <= worst)) worst = m;
        }
    std::printf("  %s %ux%ux%u %s %s: metric %.3e (limit %.0e)\n", cplx ? "cplxf" : (O::type == de::_FP16_ ? "fp16" : "fp32"),
                M, N, K, fused ? "fused" : "plain", host_overload ? "host-matrix" : "device-matrix", worst, O::tol);
    CHECK(worst <= O::tol);
    A.release(); B.release(); C.release(); D.release();
}

// the reference sample's known answer: A = (j, 0), B = (i, 0), C = (1e6, 1e6) -> (sum i^2 + 1e6, 1e6)
static void sample_known_answer() {
    const uint32_t W = 1013, H = 1077, L = 1005;
    de::Matrix& A = de::CreateMatrixRef(de::_COMPLEX_F32_, L, H);
    de::Matrix& B = de::CreateMatrixRef(de::_COMPLEX_F32_, W, L);
    de::Matrix& C = de::CreateMatrixRef(de::_COMPLEX_F32_, W, H);
    de::Matrix& D = de::CreateMatrixRef(de::_COMPLEX_F32_, W, H);
    for (uint32_t i = 0; i < H; ++i) for (uint32_t j = 0; j < L; ++j) *A.ptr<de::CPf>(i, j) = de::CPf(float(j), 0.f);
    for (uint32_t i = 0; i < L; ++i) for (uint32_t j = 0; j < W; ++j) *B.ptr<de::CPf>(i, j) = de::CPf(float(i), 0.f);
    for (uint32_t i = 0; i < H; ++i) for (uint32_t j = 0; j < W; ++j) *C.ptr<de::CPf>(i, j) = de::CPf(1e6f, 1e6f);
    de::GPU_Matrix& dA = de::CreateGPUMatrixRef(de::_COMPLEX_F32_, L, H);
    de::GPU_Matrix& dB = de::CreateGPUMatrixRef(de::_COMPLEX_F32_, W, L);
    de::GPU_Matrix& dC = de::CreateGPUMatrixRef(de::_COMPLEX_F32_, W, H);
    de::GPU_Matrix& dD = de::CreateGPUMatrixRef(de::_COMPLEX_F32_, W, H);
    de::Memcpy(A, dA, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(L, H), de::DECX_MEMCPY_H2D);
    de::Memcpy(B, dB, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(W, L), de::DECX_MEMCPY_H2D);
    de::Memcpy(C, dC, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(W, H), de::DECX_MEMCPY_H2D);
    de::blas::cuda::GEMM(dA, dB, dC, dD, de::Number(de::CPf(1.f, 0.f)), de::Number(de::CPf(1.f, 0.f)));
    de::Memcpy(D, dD, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(W, H), de::DECX_MEMCPY_D2H);
    double expect = 1e6;
    for (uint32_t i = 0; i < L; ++i) expect += double(i) * i;
    double worst = 0;
    for (uint32_t i = 0; i < H; ++i) for (uint32_t j = 0; j < W; ++j) {
        worst = std::fmax(worst, std::fabs(D.ptr<de::CPf>(i, j)->real - expect) / expect);
        worst = std::fmax(worst, std::fabs(D.ptr<de::CPf>(i, j)->image - 1e6) / expect);
    }
    std::printf("  sample known answer: worst relative deviation %.3e\n", worst);
    CHECK(worst < 2e-6);
}

static void error_paths() {
    de::GPU_Matrix& a = de::CreateGPUMatrixRef(de::_FP32_, 8, 4);     // 4 x 8
    de::GPU_Matrix& b = de::CreateGPUMatrixRef(de::_FP32_, 5, 9);     // 9 x 5: inner extents differ
    de::GPU_Matrix& h = de::CreateGPUMatrixRef(de::_FP16_, 5, 8);
    de::GPU_Matrix& d = de::CreateGPUMatrixRef();
    de::ResetLastError();
    de::blas::cuda::GEMM(a, b, d);
    CHECK(de::GetLastError()->error_type == de::DECX_FAIL_DimsNotMatching);
    de::ResetLastError();
    de::blas::cuda::GEMM(a, h, d);
    CHECK(de::GetLastError()->error_type == de::DECX_FAIL_TYPE_MOT_MATCH);
    de::GPU_Matrix& b2 = de::CreateGPUMatrixRef(de::_FP32_, 5, 8);
    de::GPU_Matrix& c2 = de::CreateGPUMatrixRef(de::_FP32_, 5, 4);
    de::ResetLastError();
    de::blas::cuda::GEMM(a, b2, c2, d, de::Number(1.0f), de::Number(de::Float2Half(1.f)));   // beta of another type
    CHECK(de::GetLastError()->error_type == de::DECX_FAIL_TYPE_MOT_MATCH);
    de::GPU_Matrix& i32 = de::CreateGPUMatrixRef(de::_INT32_, 8, 8);
    de::ResetLastError();
    de::blas::cuda::GEMM(i32, i32, d);
    CHECK(de::GetLastError()->error_type == de::DECX_FAIL_UNSUPPORTED_TYPE);
    de::ResetLastError();
    de::blas::cuda::GEMM(a, b2, a);                                   // dst aliases a factor
    CHECK(de::GetLastError()->error_type == de::DECX_FAIL_INVALID_PARAM);
    // Memcpy range check: {x = column, y = row}
    de::Matrix& hm = de::CreateMatrixRef(de::_FP32_, 8, 4);
    de::ResetLastError();
    de::DH r = de::Memcpy(hm, a, de::Point2D(4, 0), de::Point2D(0, 0), de::Point2D(8, 4), de::DECX_MEMCPY_H2D);
    CHECK(r.error_type == de::DECX_FAIL_MEMCPY_OVERRANGED);
    // sub-block copy lands where it should
    for (int i = 0; i < 4; ++i) for (int j = 0; j < 8; ++j) *hm.ptr<float>(i, j) = float(10 * i + j);
    de::Matrix& back = de::CreateMatrixRef(de::_FP32_, 8, 4);
    r = de::Memcpy(hm, a, de::Point2D(2, 1), de::Point2D(1, 0), de::Point2D(3, 2), de::DECX_MEMCPY_H2D);
    CHECK(r.error_type == de::DECX_SUCCESS);
    de::Memcpy(back, a, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(8, 4), de::DECX_MEMCPY_D2H);
    CHECK(*back.ptr<float>(0, 1) == 12.f && *back.ptr<float>(1, 3) == 24.f && *back.ptr<float>(0, 0) == 0.f);
    // dst is grown on demand and keeps its block when the next result is smaller
    de::GPU_Matrix& big = de::CreateGPUMatrixRef(de::_FP32_, 64, 64);
    de::ResetLastError();
    de::blas::cuda::GEMM(big, big, d);
    CHECK(d.Width() == 64 && d.Height() == 64 && de::GetLastError()->error_type == de::DECX_SUCCESS);
    de::blas::cuda::GEMM(a, b2, d);
    CHECK(d.Width() == 5 && d.Height() == 4 && de::GetLastError()->error_type == de::DECX_SUCCESS);
}

// Vector overloads of GEMM (host objects), every accumulation level
static void gemv_cases() {
    const uint32_t shapes[][2] = {{1, 1}, {37, 129}, {300, 4099}, {2050, 515}};      // rows, cols of the matrix
    for (auto& sh : shapes) {
        const uint32_t rows = sh[0], cols = sh[1];
        for (int trans = 0; trans < 2; ++trans) {
            const uint32_t nin = trans ? rows : cols, nout = trans ? cols : rows;
            // fp32
            de::Matrix& A = de::CreateMatrixRef(de::_FP32_, cols, rows);
            de::Vector& x = de::CreateVectorRef(de::_FP32_, nin);
            de::Vector& y = de::CreateVectorRef();
            for (uint32_t i = 0; i < rows; ++i) for (uint32_t j = 0; j < cols; ++j) *A.ptr<float>(i, j) = rnd();
            for (uint32_t i = 0; i < nin; ++i) *x.ptr<float>(i) = rnd();
            if (trans) de::blas::cuda::GEMM(x, A, y); else de::blas::cuda::GEMM(A, x, y);
            CHECK(de::GetLastError()->error_type == de::DECX_SUCCESS && y.Len() == nout && y.Type() == de::_FP32_);
            double worst = 0;
            for (uint32_t o = 0; o < nout; ++o) {
                double s = 0, na = 0, nx = 0;
                for (uint32_t k = 0; k < nin; ++k) {
                    const double a = trans ? *A.ptr<float>(k, o) : *A.ptr<float>(o, k), v = *x.ptr<float>(k);
                    s += a * v; na += a * a; nx += v * v;
                }
                worst = std::fmax(worst, std::fabs(*y.ptr<float>(o) - s) / (std::sqrt(na * nx) + 1e-300));
            }
            CHECK(worst <= 1e-5);
            A.release(); x.release(); y.release();
            // fp16, three levels
            for (uint32_t accu = 0; accu < 3; ++accu) {
                de::Matrix& Ah = de::CreateMatrixRef(de::_FP16_, cols, rows);
                de::Vector& xh = de::CreateVectorRef(de::_FP16_, nin);
                de::Vector& yh = de::CreateVectorRef();
                for (uint32_t i = 0; i < rows; ++i) for (uint32_t j = 0; j < cols; ++j) *Ah.ptr<de::Half>(i, j) = de::Float2Half(rnd() * 0.1f);
                for (uint32_t i = 0; i < nin; ++i) *xh.ptr<de::Half>(i) = de::Float2Half(rnd() * 0.1f);
                if (trans) de::blas::cuda::GEMM(xh, Ah, yh, accu); else de::blas::cuda::GEMM(Ah, xh, yh, accu);
                CHECK(de::GetLastError()->error_type == de::DECX_SUCCESS && yh.Len() == nout);
                CHECK(yh.Type() == (accu == 0 ? de::_FP32_ : de::_FP16_));
                worst = 0;
                for (uint32_t o = 0; o < nout; ++o) {
                    double s = 0, na = 0, nx = 0;
                    for (uint32_t k = 0; k < nin; ++k) {
                        const double a = de::Half2Float(trans ? *Ah.ptr<de::Half>(k, o) : *Ah.ptr<de::Half>(o, k));
                        const double v = de::Half2Float(*xh.ptr<de::Half>(k));
                        s += a * v; na += a * a; nx += v * v;
                    }
                    const double got = accu == 0 ? double(*yh.ptr<float>(o)) : double(de::Half2Float(*yh.ptr<de::Half>(o)));
                    worst = std::fmax(worst, (std::fabs(got - s) - 3e-8) / (std::sqrt(na * nx) + 1e-300));
                }
                CHECK(worst <= 1e-2);
                Ah.release(); xh.release(); yh.release();
            }
        }
    }
    // error paths
    de::Matrix& A = de::CreateMatrixRef(de::_FP32_, 8, 4);
    de::Vector& bad = de::CreateVectorRef(de::_FP32_, 5);
    de::Vector& y = de::CreateVectorRef();
    de::blas::cuda::GEMM(A, bad, y);
    CHECK(de::GetLastError()->error_type == de::DECX_FAIL_DimsNotMatching);
    de::Vector& h = de::CreateVectorRef(de::_FP16_, 8);
    de::blas::cuda::GEMM(A, h, y);
    CHECK(de::GetLastError()->error_type == de::DECX_FAIL_TYPE_MOT_MATCH);
}

// de::cuda::Transpose and de::cuda::TypeCast on device matrices, then the fp16 GEMM on the cast operands
static void transpose_cast_cases() {
    const uint32_t W = 301, H = 130;
    de::Matrix& hm = de::CreateMatrixRef(de::_FP32_, W, H);
    for (uint32_t i = 0; i < H; ++i) for (uint32_t j = 0; j < W; ++j) *hm.ptr<float>(i, j) = rnd();
    de::GPU_Matrix& g = de::CreateGPUMatrixRef(de::_FP32_, W, H);
    de::Memcpy(hm, g, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(W, H), de::DECX_MEMCPY_H2D);
    de::GPU_Matrix& gt = de::CreateGPUMatrixRef();
    de::DH r = de::cuda::Transpose(g, gt);
    CHECK(r.error_type == de::DECX_SUCCESS && gt.Width() == H && gt.Height() == W && gt.Type() == de::_FP32_);
    de::Matrix& back = de::CreateMatrixRef(de::_FP32_, H, W);
    de::Memcpy(back, gt, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(H, W), de::DECX_MEMCPY_D2H);
    bool same = true;
    for (uint32_t i = 0; i < H; ++i) for (uint32_t j = 0; j < W; ++j) same = same && (*back.ptr<float>(j, i) == *hm.ptr<float>(i, j));
    CHECK(same);
    // fp32 -> fp16 on the device equals the host conversion bit for bit; and back is exact
    de::GPU_Matrix& gh = de::CreateGPUMatrixRef();
    r = de::cuda::TypeCast(g, gh, de::CVT_FP32_FP16);
    CHECK(r.error_type == de::DECX_SUCCESS && gh.Type() == de::_FP16_ && gh.Width() == W && gh.Height() == H);
    de::Matrix& hh = de::CreateMatrixRef(de::_FP16_, W, H);
    de::Memcpy(hh, gh, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(W, H), de::DECX_MEMCPY_D2H);
    same = true;
    for (uint32_t i = 0; i < H; ++i) for (uint32_t j = 0; j < W; ++j) same = same && (hh.ptr<de::Half>(i, j)->val == de::Float2Half(*hm.ptr<float>(i, j)).val);
    CHECK(same);
    de::GPU_Matrix& g2 = de::CreateGPUMatrixRef();
    r = de::cuda::TypeCast(gh, g2, de::CVT_FP16_FP32);
    CHECK(r.error_type == de::DECX_SUCCESS && g2.Type() == de::_FP32_);
    de::Matrix& h2 = de::CreateMatrixRef(de::_FP32_, W, H);
    de::Memcpy(h2, g2, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(W, H), de::DECX_MEMCPY_D2H);
    same = true;
    for (uint32_t i = 0; i < H; ++i) for (uint32_t j = 0; j < W; ++j) same = same && (*h2.ptr<float>(i, j) == de::Half2Float(*hh.ptr<de::Half>(i, j)));
    CHECK(same);
    // fp32 <-> fp64
    de::GPU_Matrix& gd = de::CreateGPUMatrixRef();
    r = de::cuda::TypeCast(g, gd, de::CVT_FP32_FP64);
    CHECK(r.error_type == de::DECX_SUCCESS && gd.Type() == de::_FP64_);
    r = de::cuda::TypeCast(gd, g2, de::CVT_FP64_FP32);
    de::Memcpy(h2, g2, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(W, H), de::DECX_MEMCPY_D2H);
    same = true;
    for (uint32_t i = 0; i < H; ++i) for (uint32_t j = 0; j < W; ++j) same = same && (*h2.ptr<float>(i, j) == *hm.ptr<float>(i, j));
    CHECK(same);
    // wrong source type / unknown method
    r = de::cuda::TypeCast(gh, g2, de::CVT_FP32_FP16);
    CHECK(r.error_type == de::DECX_FAIL_TYPE_MOT_MATCH);
    r = de::cuda::TypeCast(g, g2, de::CVT_UINT8_CYCLIC);
    CHECK(r.error_type == de::DECX_FAIL_INVALID_PARAM);
    // the cast operand feeds the fp16 GEMM: (H x W) . (W x H)
    de::GPU_Matrix& ght = de::CreateGPUMatrixRef();
    de::cuda::Transpose(gh, ght);
    de::GPU_Matrix& prod = de::CreateGPUMatrixRef();
    de::ResetLastError();
    de::blas::cuda::GEMM(gh, ght, prod);
    CHECK(de::GetLastError()->error_type == de::DECX_SUCCESS && prod.Width() == H && prod.Height() == H);
    de::Matrix& hp = de::CreateMatrixRef(de::_FP16_, H, H);
    de::Memcpy(hp, prod, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(H, H), de::DECX_MEMCPY_D2H);
    double worst = 0;
    for (uint32_t i = 0; i < H; i += 7)
        for (uint32_t j = 0; j < H; j += 5) {
            double s = 0, na = 0, nb = 0;
            for (uint32_t k = 0; k < W; ++k) {
                const double a = de::Half2Float(*hh.ptr<de::Half>(i, k)), b = de::Half2Float(*hh.ptr<de::Half>(j, k));
                s += a * b; na += a * a; nb += b * b;
            }
            worst = std::fmax(worst, std::fabs(de::Half2Float(*hp.ptr<de::Half>(i, j)) - s) / std::sqrt(na * nb));
        }
    CHECK(worst <= 1e-2);
}

// Host-matrix fp16 GEMM large enough (threshold lowered through the environment) to be sharded over every visible GPU
static void multi_gpu_host_case() {
    setenv("DECX_B200_MULTI_MIN_FLOPS", "1e9", 1);
    const uint32_t M = 1300, N = 2104, K = 520;
    de::Matrix& A = de::CreateMatrixRef(de::_FP16_, K, M);
    de::Matrix& B = de::CreateMatrixRef(de::_FP16_, N, K);
    de::Matrix& D = de::CreateMatrixRef();
    for (uint32_t i = 0; i < M; ++i) for (uint32_t j = 0; j < K; ++j) *A.ptr<de::Half>(i, j) = de::Float2Half(rnd() * 0.2f);
    for (uint32_t i = 0; i < K; ++i) for (uint32_t j = 0; j < N; ++j) *B.ptr<de::Half>(i, j) = de::Float2Half(rnd() * 0.2f);
    de::cuda::PinMemory(A);
    de::cuda::PinMemory(B);
    de::ResetLastError();
    de::blas::cuda::GEMM(A, B, D);
    CHECK(de::GetLastError()->error_type == de::DECX_SUCCESS && D.Width() == N && D.Height() == M);
    double worst = 0;
    for (uint32_t i = 0; i < M; i += 13)
        for (uint32_t j = 0; j < N; j += 31) {
            double s = 0, na = 0, nb = 0;
            for (uint32_t k = 0; k < K; ++k) {
                const double a = de::Half2Float(*A.ptr<de::Half>(i, k)), b = de::Half2Float(*B.ptr<de::Half>(k, j));
                s += a * b; na += a * a; nb += b * b;
            }
            worst = std::fmax(worst, std::fabs(de::Half2Float(*D.ptr<de::Half>(i, j)) - s) / std::sqrt(na * nb));
        }
    CHECK(worst <= 1e-2);
    // the same product on one GPU gives the same bits
    setenv("DECX_B200_MULTI_MIN_FLOPS", "1e30", 1);
    de::Matrix& D1 = de::CreateMatrixRef();
    de::blas::cuda::GEMM(A, B, D1);
    bool same = de::GetLastError()->error_type == de::DECX_SUCCESS;
    for (uint32_t i = 0; i < M && same; ++i) for (uint32_t j = 0; j < N; ++j) same = same && (D.ptr<de::Half>(i, j)->val == D1.ptr<de::Half>(i, j)->val);
    CHECK(same);
    unsetenv("DECX_B200_MULTI_MIN_FLOPS");
}

// Four host threads multiply different shapes and types at once: each call has its own stream, scratch and
// status word, so they overlap on the GPU and none may disturb another's result.
static void concurrent_calls() {
    struct Job { uint32_t M, N, K; bool half; };
    const Job jobs[4] = {{700, 300, 520, false}, {257, 1031, 129, false}, {900, 520, 256, true}, {1300, 136, 700, false}};
    std::vector<double> worst(4, 1e9);
    std::vector<std::thread> th;
    for (int t = 0; t < 4; ++t)
        th.emplace_back([&, t] {
            const Job j = jobs[t];
            const de::_DATA_TYPES_FLAGS_ ty = j.half ? de::_FP16_ : de::_FP32_;
            de::Matrix& A = de::CreateMatrixRef(ty, j.K, j.M);
            de::Matrix& B = de::CreateMatrixRef(ty, j.N, j.K);
            de::Matrix& D = de::CreateMatrixRef(ty, j.N, j.M);
            uint32_t seed = 77 + t;
            auto r = [&] { seed = seed * 1664525u + 1013904223u; return float(int32_t(seed >> 8) - (1 << 23)) / float(1 << 23); };
            for (uint32_t i = 0; i < j.M; ++i) for (uint32_t k = 0; k < j.K; ++k) { if (j.half) *A.ptr<de::Half>(i, k) = de::Float2Half(r() * 0.3f); else *A.ptr<float>(i, k) = r(); }
            for (uint32_t k = 0; k < j.K; ++k) for (uint32_t c = 0; c < j.N; ++c) { if (j.half) *B.ptr<de::Half>(k, c) = de::Float2Half(r() * 0.3f); else *B.ptr<float>(k, c) = r(); }
            de::GPU_Matrix& dA = de::CreateGPUMatrixRef(ty, j.K, j.M);
            de::GPU_Matrix& dB = de::CreateGPUMatrixRef(ty, j.N, j.K);
            de::GPU_Matrix& dD = de::CreateGPUMatrixRef();
            de::Memcpy(A, dA, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(j.K, j.M), de::DECX_MEMCPY_H2D);
            de::Memcpy(B, dB, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(j.N, j.K), de::DECX_MEMCPY_H2D);
            for (int rep = 0; rep < 8; ++rep) de::blas::cuda::GEMM(dA, dB, dD);
            de::Memcpy(D, dD, de::Point2D(0, 0), de::Point2D(0, 0), de::Point2D(j.N, j.M), de::DECX_MEMCPY_D2H);
            double w = 0;
            for (uint32_t i = 0; i < j.M; i += 7)
                for (uint32_t c = 0; c < j.N; c += 5) {
                    double s = 0, na = 0, nb = 0;
                    for (uint32_t k = 0; k < j.K; ++k) {
                        const double a = j.half ? de::Half2Float(*A.ptr<de::Half>(i, k)) : *A.ptr<float>(i, k);
                        const double b = j.half ? de::Half2Float(*B.ptr<de::Half>(k, c)) : *B.ptr<float>(k, c);
                        s += a * b; na += a * a; nb += b * b;
                    }
                    const double got = j.half ? de::Half2Float(*D.ptr<de::Half>(i, c)) : *D.ptr<float>(i, c);
                    w = std::fmax(w, std::fabs(got - s) / std::sqrt(na * nb));
                }
            worst[t] = w / (j.half ? 1e-2 : 1e-5);
            dA.release(); dB.release(); dD.release();
        });
    for (auto& t : th) t.join();
    for (int t = 0; t < 4; ++t) CHECK(worst[t] <= 1.0);
}

// de::nn::cuda::Conv2D, the way samples/Conv2D/Conv2D.cpp drives it: host tensor and tensor array filled through
// ptr<T>(), uploaded with de::Memcpy (the kernels slice by slice through Extract_SoftCopy), result downloaded and
// compared with the direct sum in double.
static void conv_case(uint32_t W, uint32_t H, uint32_t C, uint32_t kw, uint32_t kh, uint32_t n, int sx, int sy,
                      de::extend_label ext) {
    de::ResetLastError();
    de::Tensor& src = de::CreateTensorRef(de::_FP32_, W, H, C);
    de::TensorArray& ker = de::CreateTensorArrayRef(de::_FP32_, kw, kh, C, n);
    for (uint32_t i = 0; i < H; ++i)
        for (uint32_t j = 0; j < W; ++j)
            for (uint32_t c = 0; c < C; ++c) *src.ptr<float>(i, j, c) = rnd();
    for (uint32_t t = 0; t < n; ++t)
        for (uint32_t i = 0; i < kh; ++i)
            for (uint32_t j = 0; j < kw; ++j)
                for (uint32_t c = 0; c < C; ++c) *ker.ptr<float>(i, j, c, t) = rnd();
    de::GPU_Tensor& dsrc = de::CreateGPUTensorRef(de::_FP32_, W, H, C);
    de::GPU_TensorArray& dker = de::CreateGPUTensorArrayRef(de::_FP32_, kw, kh, C, n);
    de::GPU_Tensor& ddst = de::CreateGPUTensorRef();
    CHECK(de::Memcpy(src, dsrc, {0, 0, 0}, {0, 0, 0}, de::Point3D(C, W, H), de::DECX_MEMCPY_H2D).error_type == de::DECX_SUCCESS);
    de::Tensor& slice = de::CreateTensorRef();
    de::GPU_Tensor& dslice = de::CreateGPUTensorRef();
    for (uint32_t t = 0; t < n; ++t) {
        CHECK(ker.Extract_SoftCopy(t, slice).error_type == de::DECX_SUCCESS);
        CHECK(dker.Extract_SoftCopy(t, dslice).error_type == de::DECX_SUCCESS);
        CHECK(de::Memcpy(slice, dslice, {0, 0, 0}, {0, 0, 0}, de::Point3D(C, kw, kh), de::DECX_MEMCPY_H2D).error_type ==
              de::DECX_SUCCESS);
    }
    const de::DH h = de::nn::cuda::Conv2D(dsrc, dker, ddst, de::Point2D(sx, sy), ext);
    CHECK(h.error_type == de::DECX_SUCCESS);
    const uint32_t py = ext == de::_EXTEND_CONSTANT_ ? kh / 2 : 0, px = ext == de::_EXTEND_CONSTANT_ ? kw / 2 : 0;
    const uint32_t OH = ext == de::_EXTEND_CONSTANT_ ? H / sy : (H - kh + 1) / sy;
    const uint32_t OW = ext == de::_EXTEND_CONSTANT_ ? W / sx : (W - kw + 1) / sx;
    const uint32_t hlim = ext == de::_EXTEND_CONSTANT_ ? OH * sy : H;
    CHECK(ddst.Width() == OW && ddst.Height() == OH && ddst.Depth() == n && ddst.Type() == de::_FP32_);
    if (h.error_type == de::DECX_SUCCESS && ddst.Width() == OW && ddst.Height() == OH) {
        de::Tensor& dst = de::CreateTensorRef(de::_FP32_, OW, OH, n);
        CHECK(de::Memcpy(dst, ddst, {0, 0, 0}, {0, 0, 0}, de::Point3D(n, OW, OH), de::DECX_MEMCPY_D2H).error_type ==
              de::DECX_SUCCESS);
        double worst = 0.0;
        for (uint32_t y = 0; y < OH; ++y)
            for (uint32_t x = 0; x < OW; ++x)
                for (uint32_t t = 0; t < n; ++t) {
                    double sum = 0.0, mag = 0.0;
                    for (uint32_t i = 0; i < kh; ++i) {
                        const int64_t yy = int64_t(y) * sy + i - py;
                        if (yy < 0 || yy >= int64_t(hlim)) continue;
                        for (uint32_t j = 0; j < kw; ++j) {
                            const int64_t xx = int64_t(x) * sx + j - px;
                            if (xx < 0 || xx >= int64_t(W)) continue;
                            for (uint32_t c = 0; c < C; ++c) {
                                const double p = double(*src.ptr<float>(int(yy), int(xx), c)) * double(*ker.ptr<float>(i, j, c, t));
                                sum += p;
                                mag += std::fabs(p);
                            }
                        }
                    }
                    const double err = std::fabs(double(*dst.ptr<float>(y, x, t)) - sum) / (mag + 1e-30);
                    if (err > worst) worst = err;
                }
        CHECK(worst <= 1e-5);
        dst.release();
    }
    // a second call with the same objects re-uses dst; a smaller problem keeps its block
    CHECK(de::nn::cuda::Conv2D(dsrc, dker, ddst, de::Point2D(sx, sy), ext).error_type == de::DECX_SUCCESS);
    src.release(); ker.release(); slice.release(); dslice.release(); dsrc.release(); dker.release(); ddst.release();
}

// tensor de::Memcpy with corners: a {D, W, H} = {3, 4, 3} block from (channel 1, column 2, row 1) of a host tensor to
// (channel 0, column 1, row 2) of a device tensor; the rest of the device tensor stays zero
static void tensor_memcpy_case() {
    de::ResetLastError();
    de::Tensor& a = de::CreateTensorRef(de::_FP32_, 10, 6, 5);
    for (uint32_t i = 0; i < 6; ++i)
        for (uint32_t j = 0; j < 10; ++j)
            for (uint32_t c = 0; c < 5; ++c) *a.ptr<float>(i, j, c) = float(100 * i + 10 * j + c + 1);
    de::GPU_Tensor& g = de::CreateGPUTensorRef(de::_FP32_, 9, 7, 6);
    CHECK(de::Memcpy(a, g, de::Point3D(1, 2, 1), de::Point3D(0, 1, 2), de::Point3D(3, 4, 3), de::DECX_MEMCPY_H2D).error_type ==
          de::DECX_SUCCESS);
    de::Tensor& b = de::CreateTensorRef(de::_FP32_, 9, 7, 6);
    CHECK(de::Memcpy(b, g, de::Point3D(0, 0, 0), de::Point3D(0, 0, 0), de::Point3D(6, 9, 7), de::DECX_MEMCPY_D2H).error_type ==
          de::DECX_SUCCESS);
    int bad = 0;
    for (uint32_t i = 0; i < 7; ++i)
        for (uint32_t j = 0; j < 9; ++j)
            for (uint32_t c = 0; c < 6; ++c) {
                const bool in = i >= 2 && i < 5 && j >= 1 && j < 5 && c < 3;
                const float want = in ? float(100 * (i - 2 + 1) + 10 * (j - 1 + 2) + (c + 1) + 1) : 0.f;
                if (*b.ptr<float>(i, j, c) != want) ++bad;
            }
    CHECK(bad == 0);
    CHECK(de::Memcpy(a, g, de::Point3D(3, 0, 0), de::Point3D(0, 0, 0), de::Point3D(3, 4, 3), de::DECX_MEMCPY_H2D).error_type ==
          de::DECX_FAIL_MEMCPY_OVERRANGED);                       // channels 3..5 of a 5-channel source
    de::GPU_Tensor& gh = de::CreateGPUTensorRef(de::_FP16_, 9, 7, 6);
    CHECK(de::Memcpy(a, gh, de::Point3D(0, 0, 0), de::Point3D(0, 0, 0), de::Point3D(1, 1, 1), de::DECX_MEMCPY_H2D).error_type ==
          de::MEMCPY_DIFFERENT_TYPES);
    a.release(); b.release(); g.release(); gh.release();
}

static void conv_cases() {
    conv_case(33, 20, 8, 3, 3, 12, 1, 1, de::_EXTEND_CONSTANT_);      // implicit form, 64-column accumulators
    conv_case(40, 31, 16, 5, 5, 4, 1, 1, de::_EXTEND_CONSTANT_);      // the sample's shape class: 5 x 5, four kernels
    conv_case(21, 17, 3, 3, 2, 5, 2, 1, de::_EXTEND_NONE_);           // odd kernel count: materialised form
    conv_case(64, 48, 32, 3, 3, 96, 1, 1, de::_EXTEND_NONE_);         // CTA pairs, 128-column accumulators
    conv_case(30, 30, 4, 7, 7, 132, 2, 2, de::_EXTEND_CONSTANT_);     // more than 128 kernels, stride 2
    // errors: depth mismatch, unsupported border mode, uninitialised operands
    de::GPU_Tensor& s = de::CreateGPUTensorRef(de::_FP32_, 8, 8, 4);
    de::GPU_TensorArray& k = de::CreateGPUTensorArrayRef(de::_FP32_, 3, 3, 8, 2);
    de::GPU_Tensor& d = de::CreateGPUTensorRef();
    CHECK(de::nn::cuda::Conv2D(s, k, d).error_type == de::DECX_FAIL_DimsNotMatching);
    de::GPU_TensorArray& k2 = de::CreateGPUTensorArrayRef(de::_FP32_, 3, 3, 4, 2);
    CHECK(de::nn::cuda::Conv2D(s, k2, d, de::Point2D(1, 1), de::_EXTEND_REFLECT_).error_type == de::DECX_FAIL_ErrorFlag);
    de::GPU_TensorArray& k3 = de::CreateGPUTensorArrayRef(de::_FP32_, 9, 9, 4, 2);
    CHECK(de::nn::cuda::Conv2D(s, k3, d).error_type == de::DECX_FAIL_DimsNotMatching);      // kernel larger than the source
    CHECK(de::nn::cuda::Conv2D(d, k2, s).error_type == de::DECX_FAIL_CLASS_NOT_INIT);
    s.release(); k.release(); k2.release(); k3.release();
}

int main() {
    de::InitCPUInfo();
    de::InitCuda();
    if (de::GetLastError()->error_type != de::DECX_SUCCESS) { std::printf("no CUDA device\n"); return 2; }
    const uint32_t shapes[][3] = {{1, 1, 1}, {17, 5, 9}, {129, 257, 65}, {300, 200, 150}, {513, 130, 260}};
    for (auto& s : shapes)
        for (int fused = 0; fused < 2; ++fused) {
            run_case<float>(s[0], s[1], s[2], fused, false);
            run_case<de::Half>(s[0], s[1], s[2], fused, false);
            run_case<de::CPf>(s[0], s[1], s[2], fused, false);
            run_case<double>(s[0], s[1], s[2], fused, false);
            run_case<de::CPd>(s[0], s[1], s[2], fused, false);
        }
    for (int fused = 0; fused < 2; ++fused) {
        run_case<float>(2300, 140, 90, fused, true);      // several row blocks in the host-matrix pipeline
        run_case<de::Half>(300, 136, 72, fused, true);
        run_case<de::CPf>(260, 70, 33, fused, true);
        run_case<double>(2100, 70, 33, fused, true);
    }
    gemv_cases();
    transpose_cast_cases();
    tensor_memcpy_case();
    conv_cases();
    multi_gpu_host_case();
    concurrent_calls();
    sample_known_answer();
    error_paths();
    de::cuda::DECX_CUDA_exit();
    if (g_fail == 0) std::printf("gemm_api: all checks passed\n");
    return g_fail == 0 ? 0 : 1;
}
