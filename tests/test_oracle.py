"""CPU tests of the parity checker itself: it must agree with the reference's golden outputs,
with the reference's only closed-form known answer, and with numpy's fp64 product."""
import os

import numpy as np
import pytest

from oracle import binding as ob

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_cpu_gemm.npz")
NAMES = ["f32_64", "f32_ragged", "f32_192", "c64_64", "c64_128x64x46", "c64_128"]


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_reference_cpu_gemm_outputs(name):
    """Golden vectors: outputs of the reference's de::blas::cpu::GEMM (tests/golden/make_golden.py).
    The reference computes in fp32, so agreement is to fp32 rounding, far inside the 1e-5 metric."""
    z = np.load(GOLD)
    A, B, D = z[name + "_A"], z[name + "_B"], z[name + "_D"]
    assert ob.metric(D, ob.gemm(A, B), A, B) < 1e-6


def test_oracle_sample_known_answer():
    """samples/Matrix_Multiplication/MatMul.cpp:64-140 of the reference: complex fused GEMM with
    A[i][j] = (j, 0), B[i][j] = (i, 0), C = (1e6, 1e6), W=1013, H=1077, L=1005; every element is
    (sum_{i<L} i^2 + 1e6, 1e6)."""
    W, H, L = 1013, 1077, 1005
    A = np.tile(np.arange(L, dtype=np.float32), (H, 1)).astype(np.complex64)
    B = np.tile(np.arange(L, dtype=np.float32)[:, None], (1, W)).astype(np.complex64)
    C = np.full((H, W), 1e6 + 1e6j, dtype=np.complex64)
    D = ob.gemm(A, B, C, 1.0, 1.0)
    expect = sum(i * i for i in range(L)) + 1e6
    assert np.all(D.real == expect) and np.all(D.imag == 1e6)


@pytest.mark.parametrize("dt", [np.float32, np.complex64])
@pytest.mark.parametrize("shape", [(1, 1, 1), (7, 5, 3), (65, 33, 129)])
def test_oracle_vs_numpy_fp64(dt, shape):
    M, N, K = shape
    rng = np.random.default_rng(5)
    mk = (lambda r, c: (rng.normal(size=(r, c)) + 1j * rng.normal(size=(r, c))).astype(dt)) if dt == np.complex64 \
        else (lambda r, c: rng.normal(size=(r, c)).astype(dt))
    A, B, C = mk(M, K), mk(K, N), mk(M, N)
    wide = np.complex128 if dt == np.complex64 else np.float64
    alpha, beta = (0.5 - 2j, 1.5 + 0.25j) if dt == np.complex64 else (0.5, -1.5)
    ref = alpha * (A.astype(wide) @ B.astype(wide)) + beta * C.astype(wide)
    assert np.allclose(ob.gemm(A, B, C, alpha, beta), ref, rtol=1e-13, atol=1e-13)
    assert np.allclose(ob.gemm(A, B), A.astype(wide) @ B.astype(wide), rtol=1e-13, atol=1e-13)


def test_oracle_fp16_accumulates_in_fp32():
    rng = np.random.default_rng(6)
    A = rng.normal(0, 0.5, (33, 70)).astype(np.float16)
    B = rng.normal(0, 0.5, (70, 41)).astype(np.float16)
    C = rng.normal(0, 0.5, (33, 41)).astype(np.float16)
    D = ob.gemm(A, B, C, 2.0, -1.0)
    assert D.dtype == np.float32
    ref = 2.0 * (A.astype(np.float64) @ B.astype(np.float64)) - C.astype(np.float64)
    assert np.abs(D - ref).max() < 1e-4
    # bit-exact sequential fp32 accumulation for one element
    acc = np.float32(0)
    for k in range(70):
        acc = np.float32(acc + np.float32(A[3, k]) * np.float32(B[k, 5]))
    assert np.float32(2.0) * acc + np.float32(-1.0) * np.float32(C[3, 5]) == D[3, 5]


def test_half_conversion_matches_ieee():
    rng = np.random.default_rng(8)
    x = (rng.normal(0, 1, 200000) * 10.0 ** rng.integers(-9, 6, 200000)).astype(np.float32)
    x[:6] = [0.0, -0.0, 65504.0, 65520.0, 5.9604645e-8, 2.9802322e-8]
    assert np.array_equal(ob.to_half(x).view(np.uint16), x.astype(np.float16).view(np.uint16))


def test_metric_properties():
    rng = np.random.default_rng(9)
    A = rng.normal(size=(9, 4)).astype(np.float32)
    B = rng.normal(size=(4, 6)).astype(np.float32)
    D = ob.gemm(A, B)
    assert ob.metric(D, D, A, B) == 0.0
    E = D.copy()
    E[2, 3] += 1e-3
    rn, cn = np.linalg.norm(A[2].astype(np.float64)), np.linalg.norm(B[:, 3].astype(np.float64))
    assert abs(ob.metric(E, D, A, B) - 1e-3 / (rn * cn)) < 1e-12
    E[0, 0] = np.nan
    assert np.isnan(ob.metric(E, D, A, B))      # NaN never passes a `<= tolerance` check


@pytest.mark.skipif(not ob.ref_available(), reason="oracle/_ref not built (reference sources not mounted)")
def test_reference_build_still_matches_golden():
    """Where the reference build exists, re-run one golden case through it."""
    z = np.load(GOLD)
    A, B, D = z["f32_64_A"], z["f32_64_B"], z["f32_64_D"]
    R, _, _ = ob.ref_cpu_gemm(A, B, threads=1)
    assert np.array_equal(R, D)
