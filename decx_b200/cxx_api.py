"""ctypes view of the C-context exports of the C++ drop-in (``decx_b200/host/libDECX_b200.so``,
``include/DECX/c_api.h``): host matrices owned by the library and ``de::blas::cuda::GEMM(de::Matrix&, ...)``.

The benchmark's end-to-end leg goes through this -- the call a DECX user makes -- and tests use it to drive the
C++ front door from Python.  There is no fallback: a missing library raises on import.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "host", "libDECX_b200.so")
if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `python -m decx_b200.build`")
lib = ctypes.CDLL(LIB_PATH)


class MatrixLayout(ctypes.Structure):
    _fields_ = [("width", ctypes.c_uint32), ("height", ctypes.c_uint32), ("pitch", ctypes.c_uint32),
                ("element_size", ctypes.c_int32)]


class Handle(ctypes.Structure):
    _fields_ = [("error_type", ctypes.c_int), ("error_string", ctypes.c_char * 100)]


vp = ctypes.c_void_p
lib.DE_CreateEmptyMatrix.restype = vp
lib.DE_CreateMatrix.restype = vp
lib.DE_CreateMatrix.argtypes = [ctypes.c_int8, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int8]
lib.DE_GetMatrixProp.restype = Handle
lib.DE_GetMatrixProp.argtypes = [vp, ctypes.POINTER(MatrixLayout)]
lib.DE_InitCuda.restype = ctypes.c_int
lib.DE_LastErrorType.restype = ctypes.c_int
lib.DE_LastErrorString.restype = ctypes.c_char_p
lib.DE_GetMatrixData.restype = vp
lib.DE_GetMatrixData.argtypes = [vp]
for f in (lib.DE_PinMatrix, lib.DE_UnpinMatrix):
    f.restype = ctypes.c_int
    f.argtypes = [vp]
lib.DE_ReleaseMatrix.restype = None
lib.DE_ReleaseMatrix.argtypes = [vp]
lib.DE_GEMM_Host.restype = ctypes.c_int
lib.DE_GEMM_Host.argtypes = [vp, vp, vp, vp]

TYPES = {np.dtype(np.float32): 1, np.dtype(np.float64): 2, np.dtype(np.float16): 3, np.dtype(np.complex64): 5,
         np.dtype(np.complex128): 6}
_NP = {v: k for k, v in TYPES.items()}


class DecxError(RuntimeError):
    def __init__(self, code):
        super().__init__(f"DECX error {code:#x}: {lib.DE_LastErrorString().decode(errors='replace')}")
        self.code = code


def init():
    rc = lib.DE_InitCuda()
    if rc != 0:
        raise DecxError(rc)


class Matrix:
    """A de::Matrix made by the library; ``array`` is a numpy view of its (pitched) storage."""

    def __init__(self, dtype=None, rows=0, cols=0, handle=None):
        self.dtype = np.dtype(dtype) if dtype is not None else None     # set it on a result before reading `array`
        self.h = handle if handle is not None else (
            lib.DE_CreateMatrix(TYPES[np.dtype(dtype)], cols, rows, 0) if dtype is not None else lib.DE_CreateEmptyMatrix())

    def layout(self):
        lay = MatrixLayout()
        lib.DE_GetMatrixProp(self.h, ctypes.byref(lay))
        return lay

    @property
    def array(self):
        lay = self.layout()
        dt = self.dtype if self.dtype is not None else np.dtype(
            {1: np.uint8, 2: np.float16, 4: np.float32, 8: np.float64, 16: np.complex128}[lay.element_size])
        n = lay.height * lay.pitch
        buf = (ctypes.c_char * (n * lay.element_size)).from_address(lib.DE_GetMatrixData(self.h))
        return np.frombuffer(buf, dtype=dt).reshape(lay.height, lay.pitch)[:, :lay.width]

    def pin(self):
        rc = lib.DE_PinMatrix(self.h)
        if rc != 0:
            raise DecxError(rc)

    def release(self):
        if self.h:
            lib.DE_ReleaseMatrix(self.h)
            self.h = None


def gemm_host(A, B, dst, C=None):
    """``de::blas::cuda::GEMM(A, B, [C,] dst)`` on host matrices; raises on a DECX error."""
    rc = lib.DE_GEMM_Host(A.h, B.h, C.h if C is not None else None, dst.h)
    if rc != 0:
        raise DecxError(rc)
