"""Device-tensor front ends of the matrix-vector product, transpose and cast entry points of the C ABI
(used by the tests and the benchmark; torch only owns memory and the stream).

Reference semantics: the Vector overloads of ``de::blas::cuda::GEMM`` (srcs/modules/BLAS/GEMM/CUDA/VMM.cu:142-184),
``de::cuda::Transpose`` (srcs/modules/BLAS/Basic_process/transpose/transpose.cu:50-101) and ``de::cuda::TypeCast``
(srcs/modules/BLAS/Basic_process/type_cast/GPU_Matrix_type_cast.cu:38-85).
"""
import ctypes

import torch

from . import capi
from .gemm import _ld

_OUT = {(capi.FP32, 0): torch.float32, (capi.FP16, capi.ACCU_L1): torch.float32,
        (capi.FP16, capi.ACCU_L2): torch.float16, (capi.FP16, capi.ACCU_L3): torch.float16}


def gemv(A, x, trans=False, fp16_accu=capi.ACCU_L1, out=None, workspace=None):
    """``y = A @ x`` (trans=False, x has A.shape[1] entries) or ``y = x @ A`` (trans=True, x has A.shape[0]).

    float32: fp32 result.  float16: ``fp16_accu`` 0 = fp32 arithmetic and an fp32 result, 1 = fp32 arithmetic and
    an fp16 result, 2 = fp16 arithmetic and an fp16 result.  Launches on torch's current stream."""
    if not A.is_cuda:
        raise RuntimeError("decx_b200.blas works on CUDA tensors only (no CPU fallback)")
    dt = {torch.float32: capi.FP32, torch.float16: capi.FP16}.get(A.dtype)
    if dt is None or x.dtype != A.dtype:
        raise TypeError("A and x must both be float32 or both float16")
    rows, cols = A.shape
    if x.numel() != (rows if trans else cols) or not x.is_contiguous():
        raise ValueError("x must be a contiguous vector matching A")
    accu = fp16_accu if dt == capi.FP16 else 0
    n = cols if trans else rows
    if out is None:
        out = torch.empty(n, dtype=_OUT[(dt, accu)], device=A.device)
    need = int(capi.lib.decxb200_gemv_workspace_bytes(dt, accu, int(trans), rows, cols))
    if need and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=A.device)
    with torch.cuda.device(A.device):
        capi.check(capi.lib.decxb200_gemv(dt, accu, int(trans), torch.cuda.current_stream().cuda_stream, rows, cols,
                                          A.data_ptr(), _ld(A), x.data_ptr(), out.data_ptr(),
                                          workspace.data_ptr() if need else None, need))
    return out


def transpose(src, out=None):
    """``out[c, r] = src[r, c]`` for a pitched 2-D tensor of 1-, 2-, 4-, 8- or 16-byte elements."""
    if not src.is_cuda:
        raise RuntimeError("decx_b200.blas works on CUDA tensors only (no CPU fallback)")
    rows, cols = src.shape
    if out is None:
        out = torch.empty((cols, rows), dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device):
        capi.check(capi.lib.decxb200_transpose(src.element_size(), torch.cuda.current_stream().cuda_stream, rows, cols,
                                               src.data_ptr(), _ld(src), out.data_ptr(), _ld(out)))
    return out


_CASTS = {(torch.float32, torch.float16): capi.CAST_F32_F16, (torch.float16, torch.float32): capi.CAST_F16_F32,
          (torch.float32, torch.float64): capi.CAST_F32_F64, (torch.float64, torch.float32): capi.CAST_F64_F32,
          (torch.int32, torch.float32): capi.CAST_I32_F32, (torch.float32, torch.int32): capi.CAST_F32_I32}


def cast(src, dtype, out=None):
    """Element type cast of a pitched 2-D tensor (fp32<->fp16, fp32<->fp64, int32<->fp32)."""
    if not src.is_cuda:
        raise RuntimeError("decx_b200.blas works on CUDA tensors only (no CPU fallback)")
    kind = _CASTS.get((src.dtype, dtype))
    if kind is None:
        raise TypeError(f"no device cast from {src.dtype} to {dtype}")
    rows, cols = src.shape
    if out is None:
        out = torch.empty((rows, cols), dtype=dtype, device=src.device)
    with torch.cuda.device(src.device):
        capi.check(capi.lib.decxb200_cast2d(kind, torch.cuda.current_stream().cuda_stream, rows, cols, src.data_ptr(),
                                            _ld(src), out.data_ptr(), _ld(out)))
    return out


def conv2d(src, kernels, strides=(1, 1), extend=0, out=None, workspace=None, status=None):
    """fp32 cross-correlation ``out[y, x, t] = sum src[y*sy+i-py, x*sx+j-px, c] * kernels[t, i, j, c]`` of an
    H x W x C tensor with n kernels of kh x kw x C (``de::nn::cuda::Conv2D``); ``extend`` 0 = no border,
    2 = zero border.  Tensors are channels-innermost and may be pitched views.  Launches on the current stream."""
    if not src.is_cuda or src.dtype != torch.float32 or kernels.dtype != torch.float32:
        raise TypeError("conv2d takes float32 CUDA tensors")
    H, W, C = src.shape
    n, kh, kw, C2 = kernels.shape
    if C2 != C or src.stride(2) != 1 or kernels.stride(3) != 1:
        raise ValueError("src is H x W x C, kernels n x kh x kw x C, channels innermost")
    sx, sy = strides
    oh, ow = ctypes.c_uint32(), ctypes.c_uint32()
    capi.check(capi.lib.decxb200_conv2d_fp32_out_dims(H, W, kh, kw, sx, sy, extend, ctypes.byref(oh), ctypes.byref(ow)))
    if out is None:
        out = torch.empty((oh.value, ow.value, n), dtype=torch.float32, device=src.device)
    src_dp, src_wp = src.stride(1), src.stride(0) // src.stride(1)
    k_dp, k_wp = kernels.stride(2), kernels.stride(1) // kernels.stride(2)
    dst_dp, dst_wp = out.stride(1), out.stride(0) // out.stride(1)
    # an odd pitch in the query selects the form that works for every destination
    need = int(capi.lib.decxb200_conv2d_fp32_workspace_bytes(H, W, C, kh, kw, n, sx, sy, extend, dst_wp,
                                                             dst_dp if out.data_ptr() % 16 == 0 else 1))
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=src.device)
    with torch.cuda.device(src.device):
        capi.check(capi.lib.decxb200_conv2d_fp32(
            torch.cuda.current_stream().cuda_stream, src.data_ptr(), H, W, C, src_wp, src_dp, kernels.data_ptr(), kh, kw, n,
            k_wp, k_dp, kernels.stride(0), out.data_ptr(), dst_wp, dst_dp, sx, sy, extend, workspace.data_ptr(), need,
            status.data_ptr() if status is not None else None))
    return out
