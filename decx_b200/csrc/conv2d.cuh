// fp32 2-D convolution as im2col + GEMM (reference: de::nn::cuda::Conv2D, srcs/modules/NN/convolution/CUDA/fp32/
// Conv2D.cu:57-131; planner cuda_conv2D_fp32_im2col_planner.cu:200-300; kernels im2col_fp32.cu, im2col_GEMM_fp32.cu).
//
// Tensors are stored channels-innermost: element (y, x, c) at base[(y * wpitch + x) * dpitch + c], the layout of
// decx::_tensor_layout (srcs/common/Classes/Tensor.h:59-82).  Like the reference the operation is a cross-correlation
// (no kernel flip):   dst(y, x, t) = sum_{i, j, c} src(y * sy + i - py, x * sx + j - px, c) * kernel_t(i, j, c)
// with (py, px) = (0, 0) and OH = (H - kh + 1) / sy, OW = (W - kw + 1) / sx for extend = none, and
// (py, px) = (kh / 2, kw / 2), zeros outside the source, OH = H / sy, OW = W / sx for extend = constant.  In that mode
// the reference's im2col also reads source rows at and below OH * sy as zeros (the bound of cu_im2col_*_BC_fp32,
// im2col_fp32.cu:132, is conv2D_area.y * strides.y + kh / 2 in extended coordinates); `Hlim` keeps that.
//
// IMPLICIT form (destination rows 16-byte aligned, kernel count a multiple of 4): the im2col matrix is never built.
// pad_split_src_kernel writes tf32 (hi, lo) planes of the source with its zero border, pack_kernels_split_kernel the
// kernels as a matrix whose rows follow (kernel row i, then the kw * Cp contiguous floats of that row), and the
// GEMM kernel's producer fetches each 128 x 32 operand tile with ONE 4-D TMA box of the planes -- (32 floats of a
// kernel row, TW output columns, kernel row i, TH output rows): neighbouring output columns are `sx` pixels apart,
// so the map's x stride is sx * Cp floats and the boxes of neighbouring columns overlap in memory -- while its
// epilogue stores (32 kernels, 32 output columns) boxes through a 3-D map of the destination tensor.
//
// MATERIALISED form (any pitch or alignment):
// Two bandwidth-bound passes build the operands of ONE dense contraction on the tensor-core path (3xTF32), already
// split into the tf32 (hi, lo) planes that contraction reads -- the fp32 im2col matrix itself is never stored:
//   im2col_split_kernel        A[m][(i * kw + j) * Cp + c], m = y * dst_wpitch + x (rows of dst's pitch padding are zero)
//   pack_kernels_split_kernel  B[(i * kw + j) * Cp + c][t]
// with Cp = C rounded up to 4 (zero channels), so that every plane store is a 16-byte store; the GEMM writes
// D = A . B straight into dst (row pitch dst_dpitch).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "prepass.cuh"

namespace dxb {

struct Conv2dGeom {
    uint32_t H, W, C, src_wpitch, src_dpitch;
    uint32_t kh, kw, sx, sy, py, px;
    uint32_t OH, OW, dst_wpitch;
    uint32_t Cp;             // C rounded up to a multiple of 4
    uint32_t Kc;             // kh * kw * Cp
    uint32_t Hlim;           // source rows >= Hlim read as zero
};

// one thread per (output position m, tap, group of 4 channels): one 16-byte load, two 16-byte stores
__global__ void im2col_split_kernel(const float* __restrict__ src, float* __restrict__ a_hi, float* __restrict__ a_lo,
                                    uint64_t ldaw, Conv2dGeom g, int vec_ok) {
    allow_dependent_launch();
    const uint32_t groups_c = g.Cp / 4;
    const uint32_t per_row = g.kh * g.kw * groups_c;
    const uint64_t rows = uint64_t(g.OH) * g.dst_wpitch;
    const uint64_t total = rows * per_row;
    for (uint64_t idx = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; idx < total; idx += uint64_t(gridDim.x) * blockDim.x) {
        const uint64_t m = idx / per_row;
        const uint32_t r = uint32_t(idx % per_row);
        const uint32_t tap = r / groups_c, c = (r % groups_c) * 4;
        const uint32_t i = tap / g.kw, j = tap % g.kw;
        const uint32_t y = uint32_t(m / g.dst_wpitch), x = uint32_t(m % g.dst_wpitch);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        const int64_t sy_ = int64_t(y) * g.sy + i - g.py, sx_ = int64_t(x) * g.sx + j - g.px;
        if (x < g.OW && sy_ >= 0 && sy_ < int64_t(g.Hlim) && sx_ >= 0 && sx_ < int64_t(g.W)) {
            const float* p = src + (uint64_t(sy_) * g.src_wpitch + uint64_t(sx_)) * g.src_dpitch + c;
            if (vec_ok && c + 4 <= g.src_dpitch) {        // the pitch padding may hold anything: masked below
                v = __ldg(reinterpret_cast<const float4*>(p));
                if (c + 1 >= g.C) v.y = 0.f;
                if (c + 2 >= g.C) v.z = 0.f;
                if (c + 3 >= g.C) v.w = 0.f;
            } else {
                v.x = p[0];
                if (c + 1 < g.C) v.y = p[1];
                if (c + 2 < g.C) v.z = p[2];
                if (c + 3 < g.C) v.w = p[3];
            }
        }
        float4 h, l;
        split1(v.x, h.x, l.x);
        split1(v.y, h.y, l.y);
        split1(v.z, h.z, l.z);
        split1(v.w, h.w, l.w);
        const uint64_t o = m * ldaw + uint64_t(tap) * g.Cp + c;
        *reinterpret_cast<float4*>(a_hi + o) = h;
        *reinterpret_cast<float4*>(a_lo + o) = l;
    }
}

// kernels: n tensors kh x kw x C (kernel_wpitch, kernel_dpitch), tensor t at kernels + t * kernel_stride (floats).
// Row k of B: kernel row i = k / row_pad, then (j, c) = the k % row_pad -th of that row's kw * Cp floats; rows with
// k % row_pad >= kw * Cp and channels c >= C are zero (row_pad = kw * Cp for the materialised im2col matrix,
// kw * Cp rounded up to 32 for the implicit form, whose k-blocks never straddle two kernel rows).
// One thread per (row k of B, group of 4 kernels).
__global__ void pack_kernels_split_kernel(const float* __restrict__ kernels, uint64_t kernel_stride, uint32_t kernel_wpitch,
                                          uint32_t kernel_dpitch, uint32_t kh, uint32_t kw, uint32_t C, uint32_t Cp, uint32_t n,
                                          uint32_t row_pad, float* __restrict__ b_hi, float* __restrict__ b_lo, uint64_t ldbw) {
    allow_dependent_launch();
    const uint32_t groups = (n + 3) / 4;
    const uint32_t row_len = kw * Cp;
    const uint64_t Kc = uint64_t(kh) * row_pad, total = Kc * groups;
    for (uint64_t idx = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; idx < total; idx += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t t = uint32_t(idx % groups) * 4;
        const uint64_t k = idx / groups;
        const uint32_t i = uint32_t(k / row_pad), rem = uint32_t(k % row_pad);
        const uint32_t j = rem / Cp, c = rem % Cp;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (rem < row_len && c < C) {
            const float* p = kernels + (uint64_t(i) * kernel_wpitch + j) * kernel_dpitch + c;
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (t + q < n) v[q] = p[uint64_t(t + q) * kernel_stride];
        }
        float4 h, l;
        split1(v[0], h.x, l.x);
        split1(v[1], h.y, l.y);
        split1(v[2], h.z, l.z);
        split1(v[3], h.w, l.w);
        *reinterpret_cast<float4*>(b_hi + k * ldbw + t) = h;
        *reinterpret_cast<float4*>(b_lo + k * ldbw + t) = l;
    }
}

// Implicit form: tf32 planes of the source with its zero border, Hp x Wp x Cp:
//   plane(yy, xx, c) = src(yy - py, xx - px, c) inside the source (rows below Hlim excluded), else 0.
// One thread per (pixel of the plane, group of 4 channels).
__global__ void pad_split_src_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo,
                                     uint32_t Hp, uint32_t Wp, Conv2dGeom g, int vec_ok) {
    allow_dependent_launch();
    const uint32_t groups_c = g.Cp / 4;
    const uint64_t total = uint64_t(Hp) * Wp * groups_c;
    for (uint64_t idx = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; idx < total; idx += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t c = uint32_t(idx % groups_c) * 4;
        const uint64_t pix = idx / groups_c;
        const uint32_t xx = uint32_t(pix % Wp), yy = uint32_t(pix / Wp);
        const int64_t sy_ = int64_t(yy) - g.py, sx_ = int64_t(xx) - g.px;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sy_ >= 0 && sy_ < int64_t(g.Hlim) && sx_ >= 0 && sx_ < int64_t(g.W)) {
            const float* p = src + (uint64_t(sy_) * g.src_wpitch + uint64_t(sx_)) * g.src_dpitch + c;
            if (vec_ok && c + 4 <= g.src_dpitch) {
                v = __ldg(reinterpret_cast<const float4*>(p));
                if (c + 1 >= g.C) v.y = 0.f;
                if (c + 2 >= g.C) v.z = 0.f;
                if (c + 3 >= g.C) v.w = 0.f;
            } else {
                v.x = p[0];
                if (c + 1 < g.C) v.y = p[1];
                if (c + 2 < g.C) v.z = p[2];
                if (c + 3 < g.C) v.w = p[3];
            }
        }
        float4 h, l;
        split1(v.x, h.x, l.x);
        split1(v.y, h.y, l.y);
        split1(v.z, h.z, l.z);
        split1(v.w, h.w, l.w);
        *reinterpret_cast<float4*>(hi + idx * 4) = h;
        *reinterpret_cast<float4*>(lo + idx * 4) = l;
    }
}

}  // namespace dxb
