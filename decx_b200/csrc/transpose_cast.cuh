// Bandwidth-bound helpers either side of a GEMM in user pipelines:
//   transpose of a pitched 2-D matrix      (reference: de::cuda::Transpose,
//       srcs/modules/BLAS/Basic_process/transpose/transpose.cu:50-101, kernels transpose2D_b1/b2/b4/b8)
//   element type casts of a pitched matrix (reference: de::cuda::TypeCast,
//       srcs/modules/BLAS/Basic_process/type_cast/GPU_Matrix_type_cast.cu:38-85: fp32<->fp64, int32->fp32;
//       the fp32<->fp16 pair is new here -- it is what produces the operands of the fp16 GEMM on the device).
// Each reads its input once and writes its output once.
#pragma once
#include <type_traits>
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

// 4-byte elements, 16-byte global accesses: a CTA moves a 64 x 64 block; a thread loads four float4 (rows 16
// apart), scatters them into the padded tile, then gathers four elements of one tile COLUMN (conflict-free with the
// 65-word row stride) into one float4 of a dst row.  Needs 16-byte aligned bases and pitches that are multiples
// of 4 elements (the caller checks); ragged edges fall back to element accesses inside the kernel.
__global__ void __launch_bounds__(256)
transpose_b4_vec_kernel(const uint32_t* __restrict__ src, uint64_t lds, uint32_t* __restrict__ dst, uint64_t ldd,
                        uint32_t rows, uint32_t cols) {
    __shared__ uint32_t tile[64][65];
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 vectors across, 16 rows down
    const uint32_t r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
#pragma unroll
    for (int i = 0; i < 64; i += 16) {
        const uint32_t r = r0 + ty + i, c = c0 + 4 * tx;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) {
            const uint32_t* p = src + uint64_t(r) * lds + c;
            if (c + 4 <= cols) v = __ldcs(reinterpret_cast<const uint4*>(p));
            else {
                if (c + 0 < cols) v.x = p[0];
                if (c + 1 < cols) v.y = p[1];
                if (c + 2 < cols) v.z = p[2];
            }
        }
        tile[ty + i][4 * tx + 0] = v.x;
        tile[ty + i][4 * tx + 1] = v.y;
        tile[ty + i][4 * tx + 2] = v.z;
        tile[ty + i][4 * tx + 3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 64; i += 16) {
        const uint32_t tc = ty + i;                                   // tile column = dst row
        const uint32_t dr = c0 + tc, dc = r0 + 4 * tx;
        if (dr >= cols || dc >= rows) continue;
        const uint4 v = make_uint4(tile[4 * tx + 0][tc], tile[4 * tx + 1][tc], tile[4 * tx + 2][tc], tile[4 * tx + 3][tc]);
        uint32_t* p = dst + uint64_t(dr) * ldd + dc;
        if (dc + 4 <= rows) __stcs(reinterpret_cast<uint4*>(p), v);
        else {
            p[0] = v.x;
            if (dc + 1 < rows) p[1] = v.y;
            if (dc + 2 < rows) p[2] = v.z;
        }
    }
}

// 2-byte elements, 16-byte global accesses.  A CTA moves 64 rows x 128 columns.  A thread loads eight elements of
// two consecutive rows (two uint4), transposes the four 2 x 2 blocks in registers -- byte_perm turns the words
// (a0 a1), (b0 b1) into (a0 b0) and (a1 b1) -- and stores the words by [column pair][row pair]; the write phase
// gathers four consecutive row pairs of one dst row into a uint4.  Needs 16-byte aligned bases and pitches that are
// multiples of 8 elements; ragged extents are handled element-wise at the edges, pitch padding is never written.
__global__ void __launch_bounds__(256)
transpose_b2_vec_kernel(const uint16_t* __restrict__ src, uint64_t lds, uint16_t* __restrict__ dst, uint64_t ldd,
                        uint32_t rows, uint32_t cols) {
    __shared__ uint32_t even[64][33], odd[64][33];     // [column pair][row pair]: words of dst rows 2cp and 2cp + 1
    const uint32_t r0 = blockIdx.y * 64, c0 = blockIdx.x * 128;
    {
        const uint32_t v = threadIdx.x & 15, rp0 = threadIdx.x >> 4;   // vector of 8 columns, row pair
#pragma unroll
        for (int i = 0; i < 32; i += 16) {
            const uint32_t rp = rp0 + i, r = r0 + 2 * rp, c = c0 + 8 * v;
            uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
            if (c < cols) {     // a vector may take in pitch padding after the last column: lds is a multiple of 8
                if (r < rows) a = __ldcs(reinterpret_cast<const uint4*>(src + uint64_t(r) * lds + c));
                if (r + 1 < rows) b = __ldcs(reinterpret_cast<const uint4*>(src + uint64_t(r + 1) * lds + c));
            }
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                even[4 * v + j][rp] = __byte_perm(aw[j], bw[j], 0x5410);
                odd[4 * v + j][rp] = __byte_perm(aw[j], bw[j], 0x7632);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t idx = threadIdx.x + 256 * i;
        const uint32_t vec = idx & 7, drow = idx >> 3;                // 8 vectors of 8 elements per dst row, 128 dst rows
        const uint32_t dr = c0 + drow, dc = r0 + 8 * vec;
        if (dr >= cols || dc >= rows) continue;
        const uint32_t (*t)[33] = (drow & 1) ? odd : even;
        const uint32_t cp = drow >> 1;
        const uint4 w = make_uint4(t[cp][4 * vec + 0], t[cp][4 * vec + 1], t[cp][4 * vec + 2], t[cp][4 * vec + 3]);
        uint16_t* p = dst + uint64_t(dr) * ldd + dc;
        if (dc + 8 <= rows) __stcs(reinterpret_cast<uint4*>(p), w);
        else {
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            for (uint32_t e = 0; e < 8 && dc + e < rows; ++e) p[e] = uint16_t(ww[e >> 1] >> (16 * (e & 1)));
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
// moves 16 bytes per access and the narrower one 8 (or 16): every load and store instruction of a warp then
// covers one contiguous span (no half-written sectors).  Vector accesses when `vec_ok`, element-wise on the tail.
template <int KIND>
__global__ void __launch_bounds__(256)
cast2d_kernel(const typename CastTypes<KIND>::S* __restrict__ src, uint64_t lds,
              typename CastTypes<KIND>::D* __restrict__ dst, uint64_t ldd, uint32_t rows, uint32_t cols, int vec_ok) {
    using S = typename CastTypes<KIND>::S;
    using D = typename CastTypes<KIND>::D;
    constexpr int WIDE = sizeof(S) > sizeof(D) ? sizeof(S) : sizeof(D);
    constexpr int G = 16 / WIDE;                                  // 4 (4-byte wide side) or 2 (8-byte wide side)
    const uint32_t groups = (cols + G - 1) / G;
    const uint64_t total = uint64_t(rows) * groups;
    const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
    constexpr int U = 4;                     // groups per thread and round: all loads are issued before the first store
    using LoadT = typename std::conditional<G * sizeof(S) == 16, uint4, uint2>::type;
    using StoreT = typename std::conditional<G * sizeof(D) == 16, uint4, uint2>::type;
    for (uint64_t i0 = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i0 < total; i0 += U * stride) {
        if (vec_ok && (cols % G) == 0 && i0 + (U - 1) * stride < total) {
            LoadT in[U];
            D* d[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint64_t i = i0 + u * stride;
                const uint32_t r = uint32_t(i / groups), c = uint32_t(i % groups) * G;
                in[u] = __ldcs(reinterpret_cast<const LoadT*>(src + uint64_t(r) * lds + c));
                d[u] = dst + uint64_t(r) * ldd + c;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const S* sv = reinterpret_cast<const S*>(&in[u]);
                D out[G];
#pragma unroll
                for (int e = 0; e < G; ++e) out[e] = cast1<KIND>(sv[e]);
                __stcs(reinterpret_cast<StoreT*>(d[u]), *reinterpret_cast<const StoreT*>(out));
            }
            continue;
        }
        for (int u = 0; u < U; ++u) {
            const uint64_t i = i0 + u * stride;
            if (i >= total) break;
            const uint32_t r = uint32_t(i / groups), c = uint32_t(i % groups) * G;
            const S* s = src + uint64_t(r) * lds + c;
            D* d = dst + uint64_t(r) * ldd + c;
            if (vec_ok && c + G <= cols) {
                S in[G];
                D out[G];
                *reinterpret_cast<LoadT*>(in) = __ldcs(reinterpret_cast<const LoadT*>(s));
#pragma unroll
                for (int e = 0; e < G; ++e) out[e] = cast1<KIND>(in[e]);
                __stcs(reinterpret_cast<StoreT*>(d), *reinterpret_cast<const StoreT*>(out));
            } else {
                for (int e = 0; e < G && c + e < cols; ++e) d[e] = cast1<KIND>(s[e]);
            }
        }
    }
}

}  // namespace dxb
