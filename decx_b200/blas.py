"""Device-tensor front ends of the matrix-vector product, transpose and cast entry points of the C ABI
(used by the tests and the benchmark; torch only owns memory and the stream).

Reference semantics: the Vector overloads of ``de::blas::cuda::GEMM`` (srcs/modules/BLAS/GEMM/CUDA/VMM.cu:142-184),
``de::cuda::Transpose`` (srcs/modules/BLAS/Basic_process/transpose/transpose.cu:50-101) and ``de::cuda::TypeCast``
(srcs/modules/BLAS/Basic_process/type_cast/GPU_Matrix_type_cast.cu:38-85).
"""
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
