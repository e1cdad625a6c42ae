"""The C-context exports of the C++ drop-in (include/DECX/c_api.h) through their ctypes view."""
import numpy as np
import pytest

from decx_b200 import cxx_api as X


def test_matrix_handles_layout_and_storage():
    for dt, esz, host_pitch in ((np.float16, 2, 16), (np.float32, 4, 8), (np.float64, 8, 8), (np.complex64, 8, 8),
                                (np.complex128, 16, 6)):
        m = X.Matrix(dt, 5, 6)                       # 5 rows, 6 columns
        lay = m.layout()
        assert (lay.width, lay.height, lay.element_size) == (6, 5, esz)
        assert lay.pitch == host_pitch and (lay.pitch * esz) % 32 == 0      # host rows start 32 bytes apart or more
        a = m.array
        assert a.shape == (5, 6) and a.dtype == np.dtype(dt) and not a.any()   # zero-filled
        a[4, 5] = 3
        assert m.array[4, 5] == 3                    # a view of the library's storage, not a copy
        m.release()
    e = X.Matrix()
    assert (e.layout().width, e.layout().height) == (0, 0)
    e.release()


def test_gemm_host_reports_through_the_error_handle_without_cuda():
    """No InitCuda was called in this process: the C++ front door must say so, not crash or compute."""
    A, B, D = X.Matrix(np.float32, 4, 4), X.Matrix(np.float32, 4, 4), X.Matrix()
    with pytest.raises(X.DecxError) as e:
        X.gemm_host(A, B, D)
    assert e.value.code == 0x16                      # DECX_FAIL_CUDA_not_init
    assert "CUDA" in str(e.value)
    assert X.lib.DE_GEMM_Host(None, B.h, None, D.h) == 0x0c      # DECX_FAIL_INVALID_PARAM
    for m in (A, B, D):
        m.release()


@pytest.mark.gpu
def test_gemm_host_through_the_c_context():
    from oracle import binding as ob
    X.init()
    rng = np.random.default_rng(1)
    M, N, K = 300, 136, 72
    for dt, tol in ((np.float32, 1e-5), (np.float16, 1e-2), (np.float64, 1e-13)):
        A, B, C, D = X.Matrix(dt, M, K), X.Matrix(dt, K, N), X.Matrix(dt, M, N), X.Matrix()
        A.array[:] = rng.uniform(-1, 1, (M, K)).astype(dt)
        B.array[:] = rng.uniform(-1, 1, (K, N)).astype(dt)
        C.array[:] = rng.uniform(-1, 1, (M, N)).astype(dt)
        A.pin()
        X.gemm_host(A, B, D)
        D.dtype = np.dtype(dt)
        a, b, c = np.ascontiguousarray(A.array), np.ascontiguousarray(B.array), np.ascontiguousarray(C.array)
        assert ob.metric(np.ascontiguousarray(D.array), ob.gemm(a, b), a, b) <= tol
        X.gemm_host(A, B, D, C)                      # dst = A.B + C
        assert ob.metric(np.ascontiguousarray(D.array), ob.gemm(a, b, c, 1.0, 1.0), a, b) <= tol
        for m in (A, B, C, D):
            m.release()
