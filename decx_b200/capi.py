"""ctypes binding of the C ABI in ``include/decx_b200.h``.

The shared library is built in-tree by ``decx_b200.build`` (nvcc, sm_100a).  There is no
fallback of any kind: if the library is missing, importing this module raises, and if a call
fails the error code is turned into ``DecxB200Error``.
"""
import ctypes
import os

FP32, FP64, FP16, CPLXF, CPLXD = 1, 2, 3, 5, 6
ACCU_L1, ACCU_L2, ACCU_L3 = 0, 1, 2
CAST_F32_F16, CAST_F16_F32, CAST_F32_F64, CAST_F64_F32, CAST_I32_F32, CAST_F32_I32 = range(6)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libdecx_b200.so")


class DecxB200Error(RuntimeError):
    def __init__(self, code, what):
        super().__init__(f"decx_b200 error {code}: {what}")
        self.code = code


class FetchJob(ctypes.Structure):
    """``decxb200_fetch_job``: one piece of B a GPU brings into its replica while the GEMM runs."""
    _fields_ = [("src", ctypes.c_void_p), ("gate", ctypes.c_void_p), ("dst", ctypes.c_void_p),
                ("notify", ctypes.c_void_p), ("row0", ctypes.c_uint32),
                ("rows", ctypes.c_uint32), ("col0", ctypes.c_uint32), ("cols", ctypes.c_uint32),
                ("panel", ctypes.c_uint32), ("publish", ctypes.c_uint32)]


def fetch_job(src, gate, row0, rows, col0, cols, panel, publish=0, dst=None, notify=None):
    """A ``decxb200_fetch_job``: pull (dst None) or push (dst = the target GPU's replica, notify = its flag)."""
    return FetchJob(src=src, gate=gate, dst=dst, notify=notify, row0=row0, rows=rows, col0=col0, cols=cols, panel=panel,
                    publish=publish)


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m decx_b200.build` "
            "(there is no CPU or PyTorch fallback for the GEMM path)")
    lib = ctypes.CDLL(LIB_PATH)
    u32, u64, vp, sz, ci = (ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int)
    lib.decxb200_gemm_workspace_bytes.restype = sz
    lib.decxb200_gemm_workspace_bytes.argtypes = [ci, u32, u32, u32]
    gemm_args = [ci, vp, u32, u32, u32, vp, u64, vp, u64, vp, u64, vp, u64, vp, vp, vp, sz, vp]
    lib.decxb200_gemm.restype = ci
    lib.decxb200_gemm.argtypes = gemm_args
    lib.decxb200_gemm_ex.restype = ci
    lib.decxb200_gemm_ex.argtypes = gemm_args + [ci, ci]
    lib.decxb200_gemm_host_arena_bytes.restype = sz
    lib.decxb200_gemm_host_arena_bytes.argtypes = [ci, u32, u32, u32, ci]
    lib.decxb200_gemm_host.restype = ci
    lib.decxb200_gemm_host.argtypes = [ci, u32, u32, u32, vp, u64, vp, u64, vp, u64, vp, u64, vp, vp, vp, sz, vp]
    lib.decxb200_gemm_host_multi_arena_bytes.restype = sz
    lib.decxb200_gemm_host_multi_arena_bytes.argtypes = [ci, ci, u32, u32, u32]
    lib.decxb200_gemm_host_multi.restype = ci
    lib.decxb200_gemm_host_multi.argtypes = [ci, ci, ctypes.POINTER(ci), u32, u32, u32, vp, u64, vp, u64, vp, u64,
                                             ctypes.POINTER(vp), sz]
    pu32 = ctypes.POINTER(u32)
    lib.decxb200_gemm_host_multi_plan.restype = ci
    lib.decxb200_gemm_host_multi_plan.argtypes = [ci, u32, u32, u32, pu32, pu32, pu32, pu32, pu32, pu32, pu32]
    lib.decxb200_gemm_fp32_noalloc.restype = ci
    lib.decxb200_gemm_fp32_noalloc.argtypes = [vp, u32, u32, u32, vp, u64, vp, u64, vp, u64, vp, u64, vp, vp, vp]
    lib.decxb200_gemm_fp16_panels.restype = ci
    lib.decxb200_gemm_fp16_panels.argtypes = [vp, u32, u32, u32, vp, u64, vp, u64, vp, u64, vp, u32,
                                              ctypes.POINTER(u32), vp, ctypes.c_uint, ci, ci]
    lib.decxb200_fetch_scratch_bytes.restype = sz
    lib.decxb200_fetch_scratch_bytes.argtypes = [u32]
    lib.decxb200_gemm_fp16_fetch.restype = ci
    lib.decxb200_gemm_fp16_fetch.argtypes = [vp, u32, u32, u32, vp, u64, vp, u64, vp, u64, vp, u32, ctypes.POINTER(u32),
                                             vp, vp, ctypes.c_uint, ctypes.POINTER(FetchJob), u32, vp, sz, ci, ci]
    lib.decxb200_gemm_fp16_fetch_staged.restype = ci
    lib.decxb200_gemm_fp16_fetch_staged.argtypes = lib.decxb200_gemm_fp16_fetch.argtypes + [vp, sz]
    lib.decxb200_fetch_d_stage_bytes.restype = sz
    lib.decxb200_fetch_d_stage_bytes.argtypes = []
    lib.decxb200_gemv_workspace_bytes.restype = sz
    lib.decxb200_gemv_workspace_bytes.argtypes = [ci, ci, ci, u32, u32]
    lib.decxb200_gemv.restype = ci
    lib.decxb200_gemv.argtypes = [ci, ci, ci, vp, u32, u32, vp, u64, vp, vp, vp, sz]
    lib.decxb200_transpose.restype = ci
    lib.decxb200_transpose.argtypes = [ci, vp, u32, u32, vp, u64, vp, u64]
    lib.decxb200_cast2d.restype = ci
    lib.decxb200_cast2d.argtypes = [ci, vp, u32, u32, vp, u64, vp, u64]
    lib.decxb200_conv2d_fp32_out_dims.restype = ci
    lib.decxb200_conv2d_fp32_out_dims.argtypes = [u32, u32, u32, u32, u32, u32, ci, ctypes.POINTER(u32), ctypes.POINTER(u32)]
    lib.decxb200_conv2d_fp32_workspace_bytes.restype = sz
    lib.decxb200_conv2d_fp32_workspace_bytes.argtypes = [u32, u32, u32, u32, u32, u32, u32, u32, ci, u32, u32]
    lib.decxb200_conv2d_fp32.restype = ci
    lib.decxb200_conv2d_fp32.argtypes = [vp, vp, u32, u32, u32, u32, u32, vp, u32, u32, u32, u32, u32, u64, vp, u32, u32,
                                         u32, u32, ci, vp, sz, vp]
    lib.decxb200_copy2d_async.restype = ci
    lib.decxb200_copy2d_async.argtypes = [vp, vp, sz, vp, sz, sz, sz]
    lib.decxb200_write_flag_async.restype = ci
    lib.decxb200_write_flag_async.argtypes = [vp, vp, ctypes.c_uint]
    pvp = ctypes.POINTER(ctypes.c_void_p)
    lib.decxb200_ipc_alloc.restype = ci
    lib.decxb200_ipc_alloc.argtypes = [sz, pvp]
    lib.decxb200_ipc_free.restype = ci
    lib.decxb200_ipc_free.argtypes = [vp]
    lib.decxb200_ipc_export.restype = ci
    lib.decxb200_ipc_export.argtypes = [vp, ctypes.c_char_p]
    lib.decxb200_ipc_open.restype = ci
    lib.decxb200_ipc_open.argtypes = [ctypes.c_char_p, pvp]
    lib.decxb200_ipc_close.restype = ci
    lib.decxb200_ipc_close.argtypes = [vp]
    lib.decxb200_last_launch_count.restype = ci
    lib.decxb200_last_launch_count.argtypes = []
    lib.decxb200_last_kernel_variant.restype = ci
    lib.decxb200_last_kernel_variant.argtypes = []
    lib.decxb200_tensor_map_cache_stats.restype = None
    lib.decxb200_tensor_map_cache_stats.argtypes = [ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_ulonglong)]
    lib.decxb200_debug_stats.restype = ci
    lib.decxb200_debug_stats.argtypes = [ctypes.POINTER(ctypes.c_ulonglong)]
    lib.decxb200_strerror.restype = ctypes.c_char_p
    lib.decxb200_strerror.argtypes = [ci]
    lib.decxb200_version.restype = ctypes.c_char_p
    lib.decxb200_version.argtypes = []
    return lib


lib = _load()

EXPORTS = [
    "decxb200_gemm_workspace_bytes", "decxb200_gemm", "decxb200_gemm_ex",
    "decxb200_gemm_host_arena_bytes", "decxb200_gemm_host", "decxb200_gemm_host_multi_arena_bytes", "decxb200_gemm_host_multi_plan",
    "decxb200_gemm_host_multi",
    "decxb200_gemm_fp32_noalloc", "decxb200_gemv_workspace_bytes", "decxb200_gemv", "decxb200_transpose",
    "decxb200_cast2d", "decxb200_conv2d_fp32_out_dims", "decxb200_conv2d_fp32_workspace_bytes", "decxb200_conv2d_fp32",
    "decxb200_gemm_fp16_panels", "decxb200_fetch_scratch_bytes", "decxb200_gemm_fp16_fetch", "decxb200_gemm_fp16_fetch_staged", "decxb200_fetch_d_stage_bytes", "decxb200_copy2d_async", "decxb200_write_flag_async",
    "decxb200_ipc_alloc", "decxb200_ipc_free", "decxb200_ipc_export", "decxb200_ipc_open", "decxb200_ipc_close",
    "decxb200_last_launch_count", "decxb200_last_kernel_variant", "decxb200_tensor_map_cache_stats", "decxb200_debug_stats", "decxb200_strerror", "decxb200_version",
]


def check(code):
    if code != 0:
        raise DecxB200Error(code, lib.decxb200_strerror(code).decode())


NOALLOC_SCRATCH_BYTES = 16 << 20


def workspace_bytes(dtype, M, N, K):
    return int(lib.decxb200_gemm_workspace_bytes(dtype, M, N, K))
