// Bandwidth-bound helpers either side of a GEMM in user pipelines:
//   transpose of a pitched 2-D matrix      (reference: de::cuda::Transpose,
//       srcs/modules/BLAS/Basic_process/transpose/transpose.cu:50-101, kernels transpose2D_b1/b2/b4/b8)
//   element type casts of a pitched matrix (reference: de::cuda::TypeCast,
//       srcs/modules/BLAS/Basic_process/type_cast/GPU_Matrix_type_cast.cu:38-85: fp32<->fp64, int32->fp32;
//       the fp32<->fp16 pair is new here -- it is what produces the operands of the fp16 GEMM on the device).
// Each reads its input once and writes its output once.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

namespace dxb {

// ---------------------------------------------------------------------------------------------- transpose
// dst[c][r] = src[r][c] for elements that are one machine word W (4, 8 or 16 bytes).  A CTA moves a TILE x TILE
// block through shared memory (padded: conflict-free both ways); global reads and writes are full rows of the tile.
template <typename W, int TILE>
__global__ void __launch_bounds__(256)
transpose_words_kernel(const W* __restrict__ src, uint64_t lds, W* __restrict__ dst, uint64_t ldd, uint32_t rows,
                       uint32_t cols) {
    __shared__ W tile[TILE][TILE + 1];
    constexpr int RSTEP = 256 / TILE;
    const uint32_t tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
    const uint32_t r0 = blockIdx.y * TILE, c0 = blockIdx.x * TILE;
#pragma unroll
    for (int i = 0; i < TILE; i += RSTEP) {
        const uint32_t r = r0 + ty + i, c = c0 + tx;
        if (r < rows && c < cols) tile[ty + i][tx] = __ldcs(src + uint64_t(r) * lds + c);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < TILE; i += RSTEP) {
        const uint32_t dr = c0 + ty + i, dc = r0 + tx;            // row / column in dst
        if (dr < cols && dc < rows) __stcs(dst + uint64_t(dr) * ldd + dc, tile[tx][ty + i]);
    }
}

// 2-byte elements: threads move 32-bit words (two elements of a row) and transpose 2 x 2 element blocks in
// registers, so that both the reads and the writes are 128-byte rows.  Needs even pitches and 4-byte aligned
// bases (the caller checks); odd extents are handled element-wise at the edges.
__global__ void __launch_bounds__(256)
transpose_b2_kernel(const uint16_t* __restrict__ src, uint64_t lds, uint16_t* __restrict__ dst, uint64_t ldd,
                    uint32_t rows, uint32_t cols) {
    // tile: 64 x 64 elements = 32 x 32 blocks of 2 x 2
    __shared__ uint32_t even[32][33], odd[32][33];    // [block column][block row]: words of dst rows 2j and 2j+1
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const uint32_t r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        const uint32_t bi = ty + i;                               // block row
        const uint32_t r = r0 + 2 * bi, c = c0 + 2 * tx;
        uint32_t w0 = 0, w1 = 0;
        if (c < cols) {
            // a word may take in the padding element after the last column: the pitch is even, so it exists
            if (r < rows) w0 = __ldcs(reinterpret_cast<const uint32_t*>(src + uint64_t(r) * lds + c));
            if (r + 1 < rows) w1 = __ldcs(reinterpret_cast<const uint32_t*>(src + uint64_t(r + 1) * lds + c));
        }
        even[tx][bi] = __byte_perm(w0, w1, 0x5410);               // (src[r][c], src[r+1][c])
        odd[tx][bi] = __byte_perm(w0, w1, 0x7632);                // (src[r][c+1], src[r+1][c+1])
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        const uint32_t bj = ty + j;                               // block column of src = pair of dst rows
        const uint32_t dc = r0 + 2 * tx;                          // dst column (= src row) of the word
        if (dc >= rows) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t dr = c0 + 2 * bj + h;
            if (dr >= cols) continue;
            const uint32_t w = h ? odd[bj][tx] : even[bj][tx];
            uint16_t* p = dst + uint64_t(dr) * ldd + dc;
            if (dc + 1 < rows) __stcs(reinterpret_cast<uint32_t*>(p), w);
            else *p = uint16_t(w & 0xffffu);                      // odd row count: the last element alone
        }
    }
}

// any element size, one element per thread (1-byte elements, or operands that miss the alignment rules above)
template <typename E>
__global__ void __launch_bounds__(256)
transpose_scalar_kernel(const E* __restrict__ src, uint64_t lds, E* __restrict__ dst, uint64_t ldd, uint32_t rows,
                        uint32_t cols) {
    __shared__ E tile[32][33];
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const uint32_t r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
#pragma unroll
    for (int i = 0; i < 32; i += 8)
        if (r0 + ty + i < rows && c0 + tx < cols) tile[ty + i][tx] = src[uint64_t(r0 + ty + i) * lds + c0 + tx];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 32; i += 8)
        if (c0 + ty + i < cols && r0 + tx < rows) dst[uint64_t(c0 + ty + i) * ldd + r0 + tx] = tile[tx][ty + i];
}

// ---------------------------------------------------------------------------------------------- casts
enum CastKind : int {
    CAST_F32_F16 = 0,   // round to nearest even; beyond the fp16 range: +-inf (IEEE), like __float2half_rn
    CAST_F16_F32 = 1,
    CAST_F32_F64 = 2,
    CAST_F64_F32 = 3,   // round to nearest even
    CAST_I32_F32 = 4,   // round to nearest even
    CAST_F32_I32 = 5,   // round to nearest even, saturating (cvt.rni.s32.f32); NaN -> 0
};

template <int KIND> struct CastTypes;
template <> struct CastTypes<CAST_F32_F16> { using S = float; using D = __half; };
template <> struct CastTypes<CAST_F16_F32> { using S = __half; using D = float; };
template <> struct CastTypes<CAST_F32_F64> { using S = float; using D = double; };
template <> struct CastTypes<CAST_F64_F32> { using S = double; using D = float; };
template <> struct CastTypes<CAST_I32_F32> { using S = int32_t; using D = float; };
template <> struct CastTypes<CAST_F32_I32> { using S = float; using D = int32_t; };

template <int KIND>
__device__ __forceinline__ typename CastTypes<KIND>::D cast1(typename CastTypes<KIND>::S v);
template <> __device__ __forceinline__ __half cast1<CAST_F32_F16>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float cast1<CAST_F16_F32>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ double cast1<CAST_F32_F64>(float v) { return double(v); }
template <> __device__ __forceinline__ float cast1<CAST_F64_F32>(double v) { return __double2float_rn(v); }
template <> __device__ __forceinline__ float cast1<CAST_I32_F32>(int32_t v) { return __int2float_rn(v); }
template <> __device__ __forceinline__ int32_t cast1<CAST_F32_I32>(float v) { return __float2int_rn(v); }

// rows x cols, pitched both sides.  A thread converts G consecutive elements, G chosen so that the wider side
// moves 32 bytes and the narrower 16 (or 8): vector accesses when `vec_ok`, element-wise on the ragged tail.
template <int KIND>
__global__ void __launch_bounds__(256)
cast2d_kernel(const typename CastTypes<KIND>::S* __restrict__ src, uint64_t lds,
              typename CastTypes<KIND>::D* __restrict__ dst, uint64_t ldd, uint32_t rows, uint32_t cols, int vec_ok) {
    using S = typename CastTypes<KIND>::S;
    using D = typename CastTypes<KIND>::D;
    constexpr int WIDE = sizeof(S) > sizeof(D) ? sizeof(S) : sizeof(D);
    constexpr int G = 32 / WIDE;                                  // 8 (4-byte wide side) or 4 (8-byte wide side)
    const uint32_t groups = (cols + G - 1) / G;
    const uint64_t total = uint64_t(rows) * groups;
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t r = uint32_t(i / groups), c = uint32_t(i % groups) * G;
        const S* s = src + uint64_t(r) * lds + c;
        D* d = dst + uint64_t(r) * ldd + c;
        if (vec_ok && c + G <= cols) {
            S in[G];
            D out[G];
            constexpr int SV = G * sizeof(S) / 16, DV = G * sizeof(D) / 16;   // 16-byte vectors per side (>= 1 ... 2)
            if constexpr (SV >= 1) {
#pragma unroll
                for (int v = 0; v < SV; ++v) reinterpret_cast<uint4*>(in)[v] = __ldcs(reinterpret_cast<const uint4*>(s) + v);
            } else {
                *reinterpret_cast<uint2*>(in) = __ldcs(reinterpret_cast<const uint2*>(s));
            }
#pragma unroll
            for (int e = 0; e < G; ++e) out[e] = cast1<KIND>(in[e]);
            if constexpr (DV >= 1) {
#pragma unroll
                for (int v = 0; v < DV; ++v) __stcs(reinterpret_cast<uint4*>(d) + v, reinterpret_cast<const uint4*>(out)[v]);
            } else {
                __stcs(reinterpret_cast<uint2*>(d), *reinterpret_cast<const uint2*>(out));
            }
        } else {
            for (int e = 0; e < G && c + e < cols; ++e) d[e] = cast1<KIND>(s[e]);
        }
    }
}

}  // namespace dxb
