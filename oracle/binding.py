"""numpy front end of oracle/gemm_oracle.c and of the reference build in oracle/_ref/.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
cpu_baseline / reference legs of bench.py -- never by the product package.
"""
import ctypes
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libdecx_ref_cpu.so")

FP32, FP16, CPLXF = 1, 3, 5


def default_ref_root():
    """Where the reference's sources are looked for: $DECX_REF_ROOT, else a checkout named `reference` beside this
    repository."""
    return os.environ.get("DECX_REF_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root=None):
    """Compile the C restatement; compile the reference's CPU GEMM too when its sources are present."""
    ref_root = ref_root or default_ref_root()
    subprocess.run(["make", "-C", HERE, "liboracle.so"], check=True, stdout=subprocess.DEVNULL)
    if os.path.isdir(os.path.join(ref_root, "srcs")):
        subprocess.run(["make", "-C", HERE, "ref", f"REF={ref_root}"], check=True, stdout=subprocess.DEVNULL)


_lib = None


def lib():
    global _lib
    if _lib is None:
        srcs = [os.path.join(HERE, f) for f in ("gemm_oracle.c", "blas_oracle.c")]
        if not os.path.exists(ORACLE_SO) or any(os.path.getmtime(f) > os.path.getmtime(ORACLE_SO) for f in srcs):
            build()
        L = ctypes.CDLL(ORACLE_SO)
        u32, sz, vp, d, f = ctypes.c_uint32, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_double, ctypes.c_float
        L.oracle_gemm_f32.argtypes = [u32, u32, u32, vp, sz, vp, sz, vp, sz, d, d, vp, sz]
        L.oracle_gemm_c32.argtypes = [u32, u32, u32, vp, sz, vp, sz, vp, sz, vp, vp, vp, sz]
        L.oracle_gemm_f16.argtypes = [u32, u32, u32, vp, sz, vp, sz, vp, sz, f, f, vp, sz]
        L.oracle_metric.restype = d
        L.oracle_metric.argtypes = [u32, u32, ctypes.c_int, vp, sz, vp, sz, vp, vp]
        L.oracle_norms_f32.argtypes = [u32, u32, u32, ctypes.c_int, vp, sz, vp, sz, vp, vp]
        L.oracle_half_to_float.argtypes = [vp, vp, sz]
        L.oracle_float_to_half.argtypes = [vp, vp, sz]
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        ci = ctypes.c_int
        L.oracle_gemv_f32.argtypes = [ci, u32, u32, vp, sz, vp, vp]
        L.oracle_gemv_f16.argtypes = [ci, u32, u32, vp, sz, vp, vp, vp, vp]
        L.oracle_conv2d_f32.argtypes = [u32, u32, u32, vp, u32, u32, u32, vp, u32, u32, ci, u32, u32, vp, vp]
        L.oracle_conv2d_f32.restype = ci
        L.oracle_gemm_f64.argtypes = [u32, u32, u32, vp, sz, vp, sz, vp, sz, d, d, vp, sz]
        L.oracle_gemm_c64.argtypes = [u32, u32, u32, vp, sz, vp, sz, vp, sz, vp, vp, vp, sz]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def gemm(A, B, C=None, alpha=1.0, beta=0.0):
    """Oracle result of D = alpha*A@B + beta*C.

    float32 -> float64 result; complex64 -> complex128 result; float16 -> float32 result
    (fp32 accumulation; the caller rounds with ``to_half`` for the stored fp16 value).
    """
    L = lib()
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    if A.dtype == np.float32:
        A, B, C = _c(A, np.float32), _c(B, np.float32), _c(C, np.float32)
        D = np.empty((M, N), dtype=np.float64)
        L.oracle_gemm_f32(M, N, K, _p(A), K, _p(B), N, _p(C), N, float(alpha), float(beta), _p(D), N)
        return D
    if A.dtype == np.complex64:
        A, B, C = _c(A, np.complex64), _c(B, np.complex64), _c(C, np.complex64)
        D = np.empty((M, N), dtype=np.complex128)
        al = np.array([complex(alpha).real, complex(alpha).imag], dtype=np.float64)
        be = np.array([complex(beta).real, complex(beta).imag], dtype=np.float64)
        L.oracle_gemm_c32(M, N, K, _p(A), K, _p(B), N, _p(C), N, _p(al), _p(be), _p(D), N)
        return D
    if A.dtype == np.float16:
        A, B, C = _c(A, np.float16), _c(B, np.float16), _c(C, np.float16)
        D = np.empty((M, N), dtype=np.float32)
        L.oracle_gemm_f16(M, N, K, _p(A), K, _p(B), N, _p(C), N, float(alpha), float(beta), _p(D), N)
        return D
    if A.dtype == np.float64:
        A, B, C = _c(A, np.float64), _c(B, np.float64), _c(C, np.float64)
        D = np.empty((M, N), dtype=np.float64)
        L.oracle_gemm_f64(M, N, K, _p(A), K, _p(B), N, _p(C), N, float(alpha), float(beta), _p(D), N)
        return D
    if A.dtype == np.complex128:
        A, B, C = _c(A, np.complex128), _c(B, np.complex128), _c(C, np.complex128)
        D = np.empty((M, N), dtype=np.complex128)
        al = np.array([complex(alpha).real, complex(alpha).imag], dtype=np.float64)
        be = np.array([complex(beta).real, complex(beta).imag], dtype=np.float64)
        L.oracle_gemm_c64(M, N, K, _p(A), K, _p(B), N, _p(C), N, _p(al), _p(be), _p(D), N)
        return D
    raise TypeError(A.dtype)


def gemv(A, x, trans=False):
    """Oracle matrix-vector product.  float32 -> float64 result.  float16 -> (fp32-accumulated result in index
    order, fp64-accumulated result, sum of |products| per output) for the three accumulation levels' checks."""
    L = lib()
    rows, cols = A.shape
    n = cols if trans else rows
    if A.dtype == np.float32:
        A, x = _c(A, np.float32), _c(x, np.float32)
        y = np.empty(n, dtype=np.float64)
        L.oracle_gemv_f32(int(trans), rows, cols, _p(A), cols, _p(x), _p(y))
        return y
    if A.dtype == np.float16:
        A, x = _c(A, np.float16), _c(x, np.float16)
        y32, y64, mag = np.empty(n, np.float32), np.empty(n, np.float64), np.empty(n, np.float64)
        L.oracle_gemv_f16(int(trans), rows, cols, _p(A), cols, _p(x), _p(y32), _p(y64), _p(mag))
        return y32, y64, mag
    raise TypeError(A.dtype)


def conv2d_dims(H, W, kh, kw, strides=(1, 1), extend=0):
    """Output (OH, OW) of the reference's Conv2D (cuda_conv2D_fp32_im2col_planner.cu:215-225)."""
    sx, sy = strides
    if extend == 0:
        return (H - kh + 1) // sy, (W - kw + 1) // sx
    return H // sy, W // sx


def conv2d(src, kernels, strides=(1, 1), extend=0):
    """Oracle cross-correlation of src (H, W, C) with kernels (n, kh, kw, C): (fp64 result (OH, OW, n), sum of
    |products| per output).  extend 0 = no border, 2 = zero border of (kh // 2, kw // 2)."""
    L = lib()
    src, kernels = _c(src, np.float32), _c(kernels, np.float32)
    H, W, C = src.shape
    n, kh, kw, _ = kernels.shape
    OH, OW = conv2d_dims(H, W, kh, kw, strides, extend)
    D, mag = np.empty((OH, OW, n), np.float64), np.empty((OH, OW, n), np.float64)
    rc = L.oracle_conv2d_f32(H, W, C, _p(src), kh, kw, n, _p(kernels), strides[0], strides[1], extend, OH, OW, _p(D), _p(mag))
    if rc != 0:
        raise ValueError("oracle_conv2d_f32: %d" % rc)
    return D, mag


def to_half(x):
    """fp32 -> fp16 with the oracle's own round-to-nearest-even conversion."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.float16)
    lib().oracle_float_to_half(_p(x), _p(out), x.size)
    return out


def metric(D, Dref, A, B):
    """max_ij |D - Dref| / (||A_i,:|| * ||B_:,j||), the parity metric of this path."""
    L = lib()
    M, K = A.shape
    N = B.shape[1]
    cplx = int(np.iscomplexobj(A))
    if A.dtype in (np.float64, np.complex128):          # 64-bit operands: norms in numpy (float32 would overflow less
        rn = np.sqrt((np.abs(A) ** 2).sum(axis=1))      # gracefully and lose the scale of tiny values)
        cn = np.sqrt((np.abs(B) ** 2).sum(axis=0))
        rn, cn = np.ascontiguousarray(rn, dtype=np.float64), np.ascontiguousarray(cn, dtype=np.float64)
    else:
        Af = np.ascontiguousarray(A.astype(np.complex64 if cplx else np.float32))
        Bf = np.ascontiguousarray(B.astype(np.complex64 if cplx else np.float32))
        rn = np.empty(M, dtype=np.float64)
        cn = np.empty(N, dtype=np.float64)
        L.oracle_norms_f32(M, N, K, cplx, _p(Af), K, _p(Bf), N, _p(rn), _p(cn))
    wide = np.complex128 if cplx else np.float64
    Dw = np.ascontiguousarray(D.astype(wide))
    Rw = np.ascontiguousarray(Dref.astype(wide))
    return float(L.oracle_metric(M, N, cplx, _p(Dw), N, _p(Rw), N, _p(rn), _p(cn)))


# ------------------------------------------------------------------ reference build (oracle/_ref)
def ref_available():
    return os.path.exists(REF_SO)


_REF_CHILD = r"""
import ctypes, json, sys
import numpy as np
so, dtype, threads, repeats, fin, fout = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5], sys.argv[6]
L = ctypes.CDLL(so)
L.decx_ref_max_threads.restype = ctypes.c_uint
z = np.load(fin)
A, B = np.ascontiguousarray(z["A"]), np.ascontiguousarray(z["B"])
M, K = A.shape; N = B.shape[1]
D = np.zeros((M, N), dtype=A.dtype)
times = np.zeros(repeats, dtype=np.float64)
threads = min(threads, int(L.decx_ref_max_threads()))
vp = ctypes.c_void_p
L.decx_ref_cpu_gemm.argtypes = [ctypes.c_int, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, vp, ctypes.c_size_t, vp,
                                ctypes.c_size_t, vp, ctypes.c_size_t, ctypes.c_uint, ctypes.c_int, vp]
rc = L.decx_ref_cpu_gemm(dtype, M, N, K, A.ctypes.data, K, B.ctypes.data, N, D.ctypes.data, N, threads, repeats,
                         times.ctypes.data)
np.savez(fout, D=D, times=times, threads=np.array([threads]), rc=np.array([rc]))
"""


def ref_cpu_gemm(A, B, threads=8, repeats=1, tmpdir=None):
    """Run the reference's de::blas::cpu::GEMM on (A, B) in a child process (one shape per process).

    Returns (D, per-call seconds, threads used).  float32 and complex64 only, plain A@B only.
    """
    import tempfile
    if not ref_available():
        raise RuntimeError("oracle/_ref/libdecx_ref_cpu.so has not been built")
    dt = FP32 if A.dtype == np.float32 else CPLXF
    with tempfile.TemporaryDirectory(dir=tmpdir) as td:
        fin, fout = os.path.join(td, "in.npz"), os.path.join(td, "out.npz")
        np.savez(fin, A=A, B=B)
        subprocess.run([sys.executable, "-c", _REF_CHILD, REF_SO, str(dt), str(threads), str(repeats), fin, fout],
                       check=True)
        z = np.load(fout)
        if int(z["rc"][0]) != 0:
            raise RuntimeError("reference harness rejected the call")
        return z["D"], z["times"], int(z["threads"][0])


_REF_TIME_CHILD = r"""
import ctypes, json, sys, time
import numpy as np
so, dtype, M, N, K, threads, repeats, seed, sigma = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5]), int(sys.argv[6]), int(sys.argv[7]), int(sys.argv[8]), float(sys.argv[9])
L = ctypes.CDLL(so)
L.decx_ref_max_threads.restype = ctypes.c_uint
rng = np.random.default_rng(seed)
def mk(r, c):
    x = rng.standard_normal((r, c), dtype=np.float32) * np.float32(sigma)
    if dtype == 5:
        x = (x + 1j * rng.standard_normal((r, c), dtype=np.float32) * np.float32(sigma)).astype(np.complex64)
    return x
A, B = mk(M, K), mk(K, N)
D = np.zeros((M, N), dtype=A.dtype)
times = np.zeros(repeats, dtype=np.float64)
threads = min(threads, int(L.decx_ref_max_threads()))
vp = ctypes.c_void_p
L.decx_ref_cpu_gemm.argtypes = [ctypes.c_int, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, vp, ctypes.c_size_t, vp,
                                ctypes.c_size_t, vp, ctypes.c_size_t, ctypes.c_uint, ctypes.c_int, vp]
rc = L.decx_ref_cpu_gemm(dtype, M, N, K, A.ctypes.data, K, B.ctypes.data, N, D.ctypes.data, N, threads, repeats,
                         times.ctypes.data)
print("REFTIME " + json.dumps({"rc": rc, "threads": threads, "times": times.tolist(), "finite": bool(np.isfinite(D).all())}))
"""


def ref_cpu_gemm_time(dtype_code, M, N, K, threads=16, repeats=2, seed=0, sigma=1.0):
    """Time the reference's de::blas::cpu::GEMM on synthetic data generated inside a child process
    (one shape per process).  Returns {"threads", "times" (seconds per call)}."""
    if not ref_available():
        raise RuntimeError("oracle/_ref/libdecx_ref_cpu.so has not been built")
    r = subprocess.run([sys.executable, "-c", _REF_TIME_CHILD, REF_SO, str(dtype_code), str(M), str(N), str(K),
                        str(threads), str(repeats), str(seed), str(sigma)], check=True, capture_output=True, text=True)
    line = [l for l in r.stdout.splitlines() if l.startswith("REFTIME ")][-1]
    res = json.loads(line[len("REFTIME "):])
    if res["rc"] != 0 or not res["finite"]:
        raise RuntimeError(f"reference harness failed: {res}")
    return res


def port_gemm_time(M, N, K, repeats=1, seed=0, sigma=1.0):
    """Time the C restatement (fp16 inputs, fp32 accumulate) -- the fallback CPU baseline where the
    reference build is absent."""
    import time
    rng = np.random.default_rng(seed)
    A = (rng.standard_normal((M, K), dtype=np.float32) * sigma).astype(np.float16)
    B = (rng.standard_normal((K, N), dtype=np.float32) * sigma).astype(np.float16)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        gemm(A, B)
        times.append(time.perf_counter() - t0)
    return {"threads": os.cpu_count() or 1, "times": times}
