// Bandwidth-bound passes that prepare fp32 / complex-fp32 operands for the 3xTF32
// tensor-core kernel.  They write into caller-provided scratch memory ("workspace").
//
// split:   x = hi + lo with hi = rn_tf32(x), lo = rn_tf32(x - hi).  Both planes hold
//          values that are exactly representable in tf32, so the result of the MMA does
//          not depend on how the tensor core would have narrowed a full fp32 operand.
//          Dropped terms (lo*lo and the rounding of lo) are <= 2^-21 relative per product.
//
// complex: an interleaved complex GEMM  D = A * B  (A: M x K, B: K x N, CPf = {re, im})
//          is the REAL product  D' = A' * B''  where
//             A'  = A viewed as M x 2K floats            (a_re, a_im, a_re, a_im, ...)
//             B'' = 2K x 2N floats,  row 2k   = ( b_re,  b_im) pairs of row k of B
//                                    row 2k+1 = (-b_im,  b_re) pairs of row k of B
//          and D' (M x 2N floats) is exactly D in interleaved storage.  This is the
//          4-real-multiplication form of the complex product in
//          srcs/modules/BLAS/GEMM/CUDA/large_squares/64b/GEMM_cplxf_B64_kernels.cu:35-44
//          (8*M*N*K real flops), laid out so the tensor-core kernel needs no complex mode.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace dxb {

// Programmatic dependent launch: the tensor-core kernel that consumes the planes may be launched with the
// "programmatic stream serialization" attribute.  Its CTAs then become resident once every CTA of the pass has
// executed this instruction (or exited) and set up their barriers and tensor memory while the pass still runs;
// they read the planes only after their own griddepcontrol.wait, which returns when the whole pass has completed
// and its writes are visible.  Without that attribute on the next launch this is a no-op.
__device__ __forceinline__ void allow_dependent_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float rn_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
// Finite x whose rounding to tf32 would overflow (|x| within 2^-11 relative of FLT_MAX) keeps the TRUNCATED
// tf32 value as hi, so hi and lo stay finite.  Non-finite x: hi = x and lo = 0 instead of inf - inf = NaN;
// the products then give inf or NaN as IEEE does, except that inf times a value whose lo plane is zero
// yields NaN (inf * 0) where a plain fp32 GEMM would keep inf -- a limit of every split-precision scheme.
__device__ __forceinline__ void split1(float x, float& hi, float& lo) {
    const uint32_t xb = __float_as_uint(x);
    const bool finite = (xb & 0x7f800000u) != 0x7f800000u;
    hi = rn_tf32(x);
    if (finite && (__float_as_uint(hi) & 0x7f800000u) == 0x7f800000u) hi = __uint_as_float(xb & 0xffffe000u);
    lo = finite ? rn_tf32(x - hi) : 0.f;
}

// X: rows x cols (ldx floats per row)  ->  hi, lo: rows x cols (ldw floats per row, ldw % 4 == 0,
// planes 16-byte aligned).  One thread per group of 4 columns.
struct SplitJob {
    const float* X;
    uint64_t ldx;
    uint32_t rows, cols;
    float *hi, *lo;
    uint64_t ldw;
    int vec_ok;
};

__device__ __forceinline__ void split_group(const SplitJob& j, uint64_t i, uint32_t groups) {
    const uint32_t r = uint32_t(i / groups);
    const uint32_t c = uint32_t(i % groups) * 4;
    const float* src = j.X + r * j.ldx + c;
    float4 v;
    if (j.vec_ok && c + 4 <= j.cols) {
        v = __ldg(reinterpret_cast<const float4*>(src));
    } else {
        v.x = (c + 0 < j.cols) ? src[0] : 0.f;
        v.y = (c + 1 < j.cols) ? src[1] : 0.f;
        v.z = (c + 2 < j.cols) ? src[2] : 0.f;
        v.w = (c + 3 < j.cols) ? src[3] : 0.f;
    }
    float4 h, l;
    split1(v.x, h.x, l.x);
    split1(v.y, h.y, l.y);
    split1(v.z, h.z, l.z);
    split1(v.w, h.w, l.w);
    *reinterpret_cast<float4*>(j.hi + r * j.ldw + c) = h;
    *reinterpret_cast<float4*>(j.lo + r * j.ldw + c) = l;
}

static __global__ void split_tf32_kernel(const float* __restrict__ X, uint64_t ldx, uint32_t rows, uint32_t cols,
                                         float* __restrict__ hi, float* __restrict__ lo, uint64_t ldw, int vec_ok) {
    allow_dependent_launch();
    const SplitJob j{X, ldx, rows, cols, hi, lo, ldw, vec_ok};
    const uint32_t groups = (cols + 3) / 4;
    const uint64_t total = uint64_t(rows) * groups;
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x)
        split_group(j, i, groups);
}

// Both operands of one product in ONE launch (small problems are launch-bound: 1024^3 spends more time between
// kernels than inside them).
static __global__ void split_tf32_pair_kernel(SplitJob a, SplitJob b) {
    allow_dependent_launch();
    const uint32_t ga = (a.cols + 3) / 4, gb = (b.cols + 3) / 4;
    const uint64_t ta = uint64_t(a.rows) * ga, total = ta + uint64_t(b.rows) * gb;
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        if (i < ta) split_group(a, i, ga);
        else split_group(b, i - ta, gb);
    }
}

// B: K x N complex (ldb complex elements per row) -> hi, lo: 2K x 2N floats (ldw floats per row).
// One thread per pair of complex columns (4 output floats per output row).
static __global__ void expand_split_cplx_b_kernel(const float2* __restrict__ B, uint64_t ldb, uint32_t K, uint32_t N,
                                           float* __restrict__ hi, float* __restrict__ lo, uint64_t ldw) {
    allow_dependent_launch();
    const uint32_t groups = (N + 1) / 2;
    const uint64_t total = uint64_t(K) * groups;
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total;
         i += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t k = uint32_t(i / groups);
        const uint32_t n = uint32_t(i % groups) * 2;
        const float2 b0 = B[k * ldb + n];
        const float2 b1 = (n + 1 < N) ? B[k * ldb + n + 1] : make_float2(0.f, 0.f);
        const float e[4] = {b0.x, b0.y, b1.x, b1.y};      // row 2k
        const float o[4] = {-b0.y, b0.x, -b1.y, b1.x};    // row 2k+1
        float4 eh, el, oh, ol;
        split1(e[0], eh.x, el.x); split1(e[1], eh.y, el.y); split1(e[2], eh.z, el.z); split1(e[3], eh.w, el.w);
        split1(o[0], oh.x, ol.x); split1(o[1], oh.y, ol.y); split1(o[2], oh.z, ol.z); split1(o[3], oh.w, ol.w);
        const uint64_t re = uint64_t(2 * k) * ldw + 2 * n;
        const uint64_t ro = re + ldw;
        *reinterpret_cast<float4*>(hi + re) = eh;
        *reinterpret_cast<float4*>(lo + re) = el;
        *reinterpret_cast<float4*>(hi + ro) = oh;
        *reinterpret_cast<float4*>(lo + ro) = ol;
    }
}

}  // namespace dxb
