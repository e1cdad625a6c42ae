"""Device-tensor front end of the C ABI, used by the tests and the benchmark.

``gemm(A, B, C, alpha, beta)`` has the meaning of the reference's
``de::blas::cuda::GEMM(GPU_Matrix& A, B, [C,] dst[, alpha, beta])``
(srcs/modules/BLAS/GEMM/CUDA/GEMM_LS.cu:315-393): ``dst = A.B`` or ``dst = alpha.A.B + beta.C`` on
row-major pitched device matrices; fp16 accumulates in fp32 and returns fp16.  torch is used only
to own device memory and the stream; the arithmetic is the library's tcgen05 kernels.
"""
import ctypes

import torch

from . import capi

_DTYPES = {torch.float32: capi.FP32, torch.float16: capi.FP16, torch.complex64: capi.CPLXF,
           torch.float64: capi.FP64, torch.complex128: capi.CPLXD}


def _ld(t):
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise ValueError("matrices must be 2-D with unit column stride (row-major, pitched)")
    return t.stride(0) if t.shape[0] > 1 else max(t.shape[1], t.stride(0))


def _scalar(dtype, v):
    if v is None:
        return None, None
    if dtype == capi.CPLXF:
        c = complex(v)
        buf = (ctypes.c_float * 2)(c.real, c.imag)
    elif dtype == capi.CPLXD:
        c = complex(v)
        buf = (ctypes.c_double * 2)(c.real, c.imag)
    elif dtype == capi.FP64:
        buf = (ctypes.c_double * 1)(float(v))
    else:
        buf = (ctypes.c_float * 1)(float(v))
    return buf, ctypes.cast(buf, ctypes.c_void_p)


def new_status(device):
    return torch.zeros(1, dtype=torch.int32, device=device)


def gemm(A, B, C=None, alpha=None, beta=None, out=None, workspace=None, status=None, cta_group=0, max_ctas=0):
    """Launch on torch's current stream of A's device; returns ``out`` (asynchronous)."""
    if not A.is_cuda:
        raise RuntimeError("decx_b200.gemm works on CUDA tensors only (no CPU fallback)")
    dt = _DTYPES.get(A.dtype)
    if dt is None or B.dtype != A.dtype or (C is not None and C.dtype != A.dtype):
        raise TypeError("A, B, C must share one dtype out of float16, float32, float64, complex64, complex128")
    M, K = A.shape
    K2, N = B.shape
    if K2 != K:
        raise ValueError(f"A is {M}x{K} but B is {K2}x{N}")
    if C is not None and tuple(C.shape) != (M, N):
        raise ValueError("C must be M x N")
    if out is None:
        out = torch.empty((M, N), dtype=A.dtype, device=A.device)
    need = capi.workspace_bytes(dt, M, N, K)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=A.device)
    with torch.cuda.device(A.device):
        stream = torch.cuda.current_stream().cuda_stream
        _a, pa = _scalar(dt, alpha)
        _b, pb = _scalar(dt, beta if C is not None else None)
        code = capi.lib.decxb200_gemm_ex(
            dt, stream, M, N, K, A.data_ptr(), _ld(A), B.data_ptr(), _ld(B),
            C.data_ptr() if C is not None else None, _ld(C) if C is not None else 0,
            out.data_ptr(), _ld(out), pa, pb,
            workspace.data_ptr() if need else None, need,
            status.data_ptr() if status is not None else None, cta_group, max_ctas)
    capi.check(code)
    return out


def host_arena_bytes(dtype, M, N, K, has_c=False):
    return int(capi.lib.decxb200_gemm_host_arena_bytes(_DTYPES[dtype], M, N, K, int(bool(has_c))))


def gemm_host(A, B, C=None, alpha=None, beta=None, out=None, arena=None, status=None, device=None):
    """Host-matrix form: A, B, C, out are CPU tensors (pin them for full PCIe speed).

    Synchronous; copies, pre-passes and GEMM are pipelined inside the library
    (``decxb200_gemm_host``).  ``arena`` is device scratch (uint8 CUDA tensor); it is allocated
    here when missing or too small.  Returns ``out``.
    """
    if A.is_cuda or B.is_cuda:
        raise RuntimeError("gemm_host takes host tensors; use gemm() for device tensors")
    if not torch.cuda.is_available():
        raise RuntimeError("decx_b200 needs a CUDA device (no CPU fallback)")
    dt = _DTYPES.get(A.dtype)
    if dt is None or B.dtype != A.dtype or (C is not None and C.dtype != A.dtype):
        raise TypeError("A, B, C must share one dtype out of float16, float32, float64, complex64, complex128")
    M, K = A.shape
    K2, N = B.shape
    if K2 != K:
        raise ValueError(f"A is {M}x{K} but B is {K2}x{N}")
    if out is None:
        out = torch.empty((M, N), dtype=A.dtype).pin_memory()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _a, pa = _scalar(dt, alpha)
    _b, pb = _scalar(dt, beta if C is not None else None)
    use_c = C is not None and beta is not None and complex(beta) != 0
    need = int(capi.lib.decxb200_gemm_host_arena_bytes(dt, M, N, K, int(use_c)))
    if arena is None or arena.numel() < need:
        arena = torch.empty(need, dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        code = capi.lib.decxb200_gemm_host(
            dt, M, N, K, A.data_ptr(), _ld(A), B.data_ptr(), _ld(B),
            C.data_ptr() if C is not None else None, _ld(C) if C is not None else 0,
            out.data_ptr(), _ld(out), pa, pb, arena.data_ptr(), need,
            status.data_ptr() if status is not None else None)
    capi.check(code)
    return out


def gemm_host_multi(A, B, out=None, devices=None, arenas=None):
    """Host-matrix fp16 GEMM sharded over several GPUs of this process (``decxb200_gemm_host_multi``).

    A, B, out: CPU tensors (pin them); ``devices``: CUDA ordinals (default: all visible); ``arenas``: one uint8
    CUDA tensor per device (allocated here when missing).  Synchronous.  Returns (out, arenas)."""
    if A.is_cuda or B.is_cuda or A.dtype != torch.float16 or B.dtype != torch.float16:
        raise TypeError("gemm_host_multi takes float16 host tensors")
    M, K = A.shape
    K2, N = B.shape
    if K2 != K:
        raise ValueError(f"A is {M}x{K} but B is {K2}x{N}")
    if devices is None:
        devices = list(range(torch.cuda.device_count()))
    if out is None:
        out = torch.empty((M, N), dtype=A.dtype).pin_memory()
    need = int(capi.lib.decxb200_gemm_host_multi_arena_bytes(capi.FP16, len(devices), M, N, K))
    if arenas is None or len(arenas) != len(devices) or any(a.numel() < need for a in arenas):
        arenas = [torch.empty(need, dtype=torch.uint8, device=torch.device("cuda", d)) for d in devices]
    devs = (ctypes.c_int * len(devices))(*devices)
    ptrs = (ctypes.c_void_p * len(devices))(*[a.data_ptr() for a in arenas])
    capi.check(capi.lib.decxb200_gemm_host_multi(capi.FP16, len(devices), devs, M, N, K, A.data_ptr(), _ld(A),
                                                 B.data_ptr(), _ld(B), out.data_ptr(), _ld(out), ptrs, need))
    return out, arenas


def gemm_raw(dt, M, N, K, a_ptr, lda, b_ptr, ldb, c_ptr, ldc, d_ptr, ldd, alpha=None, beta=None,
             ws_ptr=None, ws_bytes=0, status_ptr=None, stream=0, cta_group=0, max_ctas=0):
    """The C ABI with raw device addresses (used where D lives in another GPU's memory)."""
    _a, pa = _scalar(dt, alpha)
    _b, pb = _scalar(dt, beta if c_ptr else None)
    capi.check(capi.lib.decxb200_gemm_ex(dt, stream, M, N, K, a_ptr, lda, b_ptr, ldb, c_ptr, ldc, d_ptr, ldd,
                                         pa, pb, ws_ptr, ws_bytes, status_ptr, cta_group, max_ctas))
    return capi.lib.decxb200_last_launch_count()


def gemm_fp16_panels(A, B, out, panel_col_end, flags, epoch, status=None, max_ctas=0, tile=0):
    """One GEMM launch over a B that arrives panel by panel (``decxb200_gemm_fp16_panels``).

    ``flags`` is an int32/uint32 CUDA tensor with one word per panel; the stream that fills panel i writes
    ``epoch`` there afterwards (``write_flag``).  Launches on torch's current stream; returns ``out``."""
    M, K = A.shape
    N = B.shape[1]
    ends = (ctypes.c_uint32 * len(panel_col_end))(*panel_col_end)
    with torch.cuda.device(A.device):
        code = capi.lib.decxb200_gemm_fp16_panels(
            torch.cuda.current_stream().cuda_stream, M, N, K, A.data_ptr(), _ld(A), B.data_ptr(), _ld(B),
            out.data_ptr(), _ld(out), status.data_ptr() if status is not None else None,
            len(panel_col_end), ends, flags.data_ptr(), epoch, max_ctas, tile)
    capi.check(code)
    return out


def gemm_fp16_fetch(A, B_replica, out_ptr, ldd, panel_col_end, ready_flags, pub_flags, epoch, jobs, scratch,
                    status=None, max_ctas=0, tile=0, d_stage=None):
    """One launch that brings B into ``B_replica`` (``jobs``: list of ``capi.FetchJob``) while it multiplies
    (``decxb200_gemm_fp16_fetch_staged``).  ``out_ptr`` is a raw device address (D may live in another GPU's
    memory); ``d_stage``: local uint8 tensor of ``decxb200_fetch_d_stage_bytes()`` bytes through which the couriers
    forward D, or None for direct stores.  Launches on torch's current stream."""
    M, K = A.shape
    N = B_replica.shape[1]
    ends = (ctypes.c_uint32 * len(panel_col_end))(*panel_col_end)
    arr = (capi.FetchJob * max(len(jobs), 1))(*jobs)
    with torch.cuda.device(A.device):
        code = capi.lib.decxb200_gemm_fp16_fetch_staged(
            torch.cuda.current_stream().cuda_stream, M, N, K, A.data_ptr(), _ld(A), B_replica.data_ptr(), _ld(B_replica),
            out_ptr, ldd, status.data_ptr() if status is not None else None, len(panel_col_end), ends,
            ready_flags.data_ptr() if ready_flags is not None else None,
            pub_flags.data_ptr() if pub_flags is not None else None, epoch, arr, len(jobs),
            scratch.data_ptr() if scratch is not None else None,
            scratch.numel() * scratch.element_size() if scratch is not None else 0, max_ctas, tile,
            d_stage.data_ptr() if d_stage is not None else None,
            d_stage.numel() * d_stage.element_size() if d_stage is not None else 0)
    capi.check(code)


def write_flag(flags, index, value, stream=None):
    """Stream-ordered store of ``value`` to ``flags[index]`` without a kernel (cuStreamWriteValue32)."""
    s = (stream or torch.cuda.current_stream(flags.device)).cuda_stream
    capi.check(capi.lib.decxb200_write_flag_async(s, flags.data_ptr() + 4 * index, value))


def copy2d(dst_ptr, dpitch, src_ptr, spitch, width_bytes, rows, stream):
    """Copy-engine 2-D copy between raw device addresses (peer mappings allowed)."""
    capi.check(capi.lib.decxb200_copy2d_async(stream.cuda_stream, dst_ptr, dpitch, src_ptr, spitch, width_bytes, rows))
