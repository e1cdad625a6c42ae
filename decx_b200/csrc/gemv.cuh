// Matrix-vector products behind the Vector overloads of de::blas::cuda::GEMM
// (reference: srcs/modules/BLAS/GEMM/CUDA/VMM.cu:55-184, kernels extreme_shapes/VMM_fp32.cu / VMM_fp16.cu,
// callers extreme_shapes/VMM_callers.cuh:67-201).
//
//   rows form   y[i] = sum_k A[i][k] * x[k]     (Matrix x Vector; the reference's "reduce_h")
//   cols form   y[j] = sum_k x[k] * A[k][j]     (Vector x Matrix; "reduce_v")
//
// Both read the matrix exactly once and are bound by HBM bandwidth; everything is organised around keeping
// many 16-byte loads in flight:
//   rows form: one warp per row and K slice; lanes stride over k with 16-byte loads of A and x (x stays in
//              L1/L2), four loads in flight per lane; shuffle reduction.
//   cols form: a thread owns 16 bytes of consecutive columns, a warp 512 contiguous bytes of a row, the
//              CTA's warps take rows k, k+W, ... of the CTA's K slice (four rows in flight per warp) and are
//              summed through shared memory.
// When the matrix has too few rows (rows form) or columns (cols form) to fill the GPU, K is cut into slices,
// each slice writes a partial vector into the workspace and gemv_finish_kernel adds them in slice order
// (deterministic, no atomics).
//
// fp16 accumulation levels of the reference (srcs/common/Classes/classes_util.h:287-300):
//   L1 (0): products and sums in fp32, fp32 result vector
//   L2 (1): products and sums in fp32, fp16 result (the reference also rounds to fp16 between its kernels)
//   L3 (2): products and sums in fp16 (hfma2) all the way, fp16 result; overflow is the caller's concern
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

namespace dxb {

constexpr int GEMV_WARPS = 8;            // warps per CTA in both forms
constexpr int GEMV_UNROLL = 4;           // 16-byte loads in flight per lane

// ---- accumulator policies ---------------------------------------------------------------------------------
struct AccF32 {                          // fp32 or fp16 inputs, fp32 arithmetic
    using part_t = float;                // type of a partial / of the value handed to the store
    static __device__ __forceinline__ float zero() { return 0.f; }
    static __device__ __forceinline__ float add(float a, float b) { return a + b; }
    static __device__ __forceinline__ float shfl_xor(float v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
};
struct AccF16 {                          // fp16 inputs, fp16 arithmetic (level L3)
    using part_t = __half;
    static __device__ __forceinline__ __half zero() { return __float2half(0.f); }
    static __device__ __forceinline__ __half add(__half a, __half b) { return __hadd(a, b); }
    static __device__ __forceinline__ __half shfl_xor(__half v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
};

template <typename OUT, typename P>
__device__ __forceinline__ OUT gemv_cast(P v);
template <> __device__ __forceinline__ float gemv_cast<float, float>(float v) { return v; }
template <> __device__ __forceinline__ __half gemv_cast<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __half gemv_cast<__half, __half>(__half v) { return v; }
template <> __device__ __forceinline__ float gemv_cast<float, __half>(__half v) { return __half2float(v); }

// dot of one 16-byte group: T = float (4 elements) or __half (8 elements)
template <typename T, typename ACC>
struct Dot16;
template <>
struct Dot16<float, AccF32> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void fma(float& acc, const uint4& a, const uint4& x) {
        acc = fmaf(__uint_as_float(a.x), __uint_as_float(x.x), acc);
        acc = fmaf(__uint_as_float(a.y), __uint_as_float(x.y), acc);
        acc = fmaf(__uint_as_float(a.z), __uint_as_float(x.z), acc);
        acc = fmaf(__uint_as_float(a.w), __uint_as_float(x.w), acc);
    }
};
template <>
struct Dot16<__half, AccF32> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void fma(float& acc, const uint4& a, const uint4& x) {
        const __half2* ah = reinterpret_cast<const __half2*>(&a);
        const __half2* xh = reinterpret_cast<const __half2*>(&x);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 af = __half22float2(ah[i]), xf = __half22float2(xh[i]);
            acc = fmaf(af.x, xf.x, acc);
            acc = fmaf(af.y, xf.y, acc);
        }
    }
};
template <>
struct Dot16<__half, AccF16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void fma(__half& acc, const uint4& a, const uint4& x) {
        const __half2* ah = reinterpret_cast<const __half2*>(&a);
        const __half2* xh = reinterpret_cast<const __half2*>(&x);
        __half2 s = __hmul2(ah[0], xh[0]);
        s = __hfma2(ah[1], xh[1], s);
        s = __hfma2(ah[2], xh[2], s);
        s = __hfma2(ah[3], xh[3], s);
        acc = __hadd(acc, __hadd(__low2half(s), __high2half(s)));
    }
};

template <typename T, typename ACC>
__device__ __forceinline__ typename ACC::part_t gemv_mul1(T a, T x);
template <> __device__ __forceinline__ float gemv_mul1<float, AccF32>(float a, float x) { return a * x; }
template <> __device__ __forceinline__ float gemv_mul1<__half, AccF32>(__half a, __half x) {
    return __half2float(a) * __half2float(x);
}
template <> __device__ __forceinline__ __half gemv_mul1<__half, AccF16>(__half a, __half x) { return __hmul(a, x); }

// ---- rows form --------------------------------------------------------------------------------------------
// grid = (ceil(M / GEMV_WARPS), slices).  out: y (slices == 1, type OUT) or partials [slice][M] of ACC::part_t.
template <typename T, typename ACC, typename OUT>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_rows_kernel(const T* __restrict__ A, uint64_t lda, const T* __restrict__ x, void* __restrict__ out,
                 uint32_t M, uint32_t K, uint32_t slice_len, int vec_ok) {
    using P = typename ACC::part_t;
    constexpr int V = Dot16<T, ACC>::N;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * GEMV_WARPS + warp;
    if (row >= M) return;
    const uint32_t k0 = blockIdx.y * slice_len;
    const uint32_t k1 = min(K, k0 + slice_len);
    const T* a = A + uint64_t(row) * lda;
    P acc = ACC::zero();
    uint32_t k = k0;
    if (vec_ok) {
        // whole 16-byte groups, GEMV_UNROLL of them in flight per lane
        const uint32_t kv_end = k0 + ((k1 - k0) / V) * V;
        for (; k + GEMV_UNROLL * 32 * V <= kv_end; k += GEMV_UNROLL * 32 * V) {
            uint4 av[GEMV_UNROLL], xv[GEMV_UNROLL];
#pragma unroll
            for (int u = 0; u < GEMV_UNROLL; ++u) {
                const uint32_t kk = k + (u * 32 + lane) * V;
                av[u] = __ldcs(reinterpret_cast<const uint4*>(a + kk));         // streamed once
                xv[u] = __ldg(reinterpret_cast<const uint4*>(x + kk));
            }
#pragma unroll
            for (int u = 0; u < GEMV_UNROLL; ++u) Dot16<T, ACC>::fma(acc, av[u], xv[u]);
        }
        for (uint32_t kk = k + lane * V; kk + V <= kv_end; kk += 32 * V) {
            const uint4 av = __ldcs(reinterpret_cast<const uint4*>(a + kk));
            const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + kk));
            Dot16<T, ACC>::fma(acc, av, xv);
        }
        k = kv_end;
    }
    for (uint32_t kk = k + lane; kk < k1; kk += 32) acc = ACC::add(acc, gemv_mul1<T, ACC>(a[kk], x[kk]));
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) acc = ACC::add(acc, ACC::shfl_xor(acc, m));
    if (lane == 0) {
        if (gridDim.y == 1) static_cast<OUT*>(out)[row] = gemv_cast<OUT, P>(acc);
        else static_cast<P*>(out)[uint64_t(blockIdx.y) * M + row] = acc;
    }
}

// ---- cols form --------------------------------------------------------------------------------------------
// grid = (ceil(N / (32 * V)), slices); x has K entries, A is K x N.
template <typename T, typename ACC, typename OUT>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_cols_kernel(const T* __restrict__ A, uint64_t lda, const T* __restrict__ x, void* __restrict__ out,
                 uint32_t K, uint32_t N, uint32_t slice_len, int vec_ok) {
    using P = typename ACC::part_t;
    constexpr int V = 16 / sizeof(T);
    __shared__ P red[GEMV_WARPS][32 * V + 1];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t col = (blockIdx.x * 32 + lane) * V;
    const uint32_t k0 = blockIdx.y * slice_len;
    const uint32_t k1 = min(K, k0 + slice_len);
    P acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = ACC::zero();
    if (col < N) {
        if (vec_ok && col + V <= N) {
            uint32_t k = k0 + warp;
            for (; k + (GEMV_UNROLL - 1) * GEMV_WARPS < k1; k += GEMV_UNROLL * GEMV_WARPS) {
                uint4 av[GEMV_UNROLL];
                T xs[GEMV_UNROLL];
#pragma unroll
                for (int u = 0; u < GEMV_UNROLL; ++u) {
                    av[u] = __ldcs(reinterpret_cast<const uint4*>(A + uint64_t(k + u * GEMV_WARPS) * lda + col));
                    xs[u] = __ldg(x + k + u * GEMV_WARPS);
                }
#pragma unroll
                for (int u = 0; u < GEMV_UNROLL; ++u) {
                    const T* e = reinterpret_cast<const T*>(&av[u]);
#pragma unroll
                    for (int i = 0; i < V; ++i) acc[i] = ACC::add(acc[i], gemv_mul1<T, ACC>(xs[u], e[i]));
                }
            }
            for (; k < k1; k += GEMV_WARPS) {
                const uint4 av = __ldcs(reinterpret_cast<const uint4*>(A + uint64_t(k) * lda + col));
                const T xk = __ldg(x + k);
                const T* e = reinterpret_cast<const T*>(&av);
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] = ACC::add(acc[i], gemv_mul1<T, ACC>(xk, e[i]));
            }
        } else {
            for (uint32_t k = k0 + warp; k < k1; k += GEMV_WARPS) {
                const T xk = x[k];
#pragma unroll
                for (int i = 0; i < V; ++i)
                    if (col + i < N) acc[i] = ACC::add(acc[i], gemv_mul1<T, ACC>(xk, A[uint64_t(k) * lda + col + i]));
            }
        }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) red[warp][lane * V + i] = acc[i];
    __syncthreads();
    // warps 0..: every thread finishes some of the CTA's 32 * V columns (summed in warp order)
    for (uint32_t c = threadIdx.x; c < 32 * V; c += GEMV_WARPS * 32) {
        const uint32_t gc = blockIdx.x * 32 * V + c;
        if (gc >= N) continue;
        P s = red[0][c];
#pragma unroll
        for (int w = 1; w < GEMV_WARPS; ++w) s = ACC::add(s, red[w][c]);
        if (gridDim.y == 1) static_cast<OUT*>(out)[gc] = gemv_cast<OUT, P>(s);
        else static_cast<P*>(out)[uint64_t(blockIdx.y) * N + gc] = s;
    }
}

// y[i] = sum over slices of partial[s][i], in slice order
template <typename ACC, typename OUT>
__global__ void gemv_finish_kernel(const typename ACC::part_t* __restrict__ partial, uint32_t slices, uint32_t n,
                                   OUT* __restrict__ y) {
    using P = typename ACC::part_t;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    P s = partial[i];
    for (uint32_t k = 1; k < slices; ++k) s = ACC::add(s, partial[uint64_t(k) * n + i]);
    y[i] = gemv_cast<OUT, P>(s);
}

}  // namespace dxb
