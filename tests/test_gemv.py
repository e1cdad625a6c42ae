"""GPU parity tests of the matrix-vector products (the Vector overloads of GEMM) through the C ABI.

fp32: against the fp64 oracle, error / (||a|| ||x||) <= 1e-5 (the path's fp32 bar; observed ~1e-7).
fp16 L1 / L2 (fp32 arithmetic): against the fp32-accumulating oracle, <= 1e-2 by the same metric -- in fact the
fp32 results agree to a few fp32 ulps of sum |a x| and L2 is that value rounded once to fp16.
fp16 L3 (fp16 arithmetic): <= 1e-2 by the metric against the fp64-accumulated value.
"""
import numpy as np
import pytest

from oracle import binding as ob

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

# (rows, cols): square, skinny both ways (sliced reductions), ragged against 4 / 8 / 32 / 128, one-element extremes
SHAPES = [(1, 1), (1, 1000), (1000, 1), (7, 5), (33, 129), (128, 128), (257, 255), (300, 4099), (4099, 300),
          (8, 70000), (70000, 8), (2048, 2048), (1023, 2050)]


@pytest.fixture(scope="module")
def Bl():
    from decx_b200 import blas
    return blas


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _pitched(t, extra):
    """Copy into a wider buffer so that the row pitch differs from the width."""
    buf = torch.full((t.shape[0], t.shape[1] + extra), float("nan"), dtype=t.dtype, device=t.device)
    buf[:, :t.shape[1]] = t
    return buf[:, :t.shape[1]]


def _scale(A, x, trans):
    a = A.astype(np.float64)
    v = x.astype(np.float64)
    if trans:
        return np.sqrt((a ** 2).sum(axis=0)) * np.linalg.norm(v) + 1e-300
    return np.sqrt((a ** 2).sum(axis=1)) * np.linalg.norm(v) + 1e-300


@pytest.mark.parametrize("trans", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemv_fp32(Bl, dev, shape, trans):
    rows, cols = shape
    rng = np.random.default_rng(rows * 3 + cols)
    A = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    x = rng.uniform(-1, 1, rows if trans else cols).astype(np.float32)
    for extra in (0, 3):                      # pitch == width (vector loads when aligned) and an odd pitch (scalar path)
        tA = _pitched(torch.from_numpy(A).to(dev), extra) if extra else torch.from_numpy(A).to(dev)
        y = Bl.gemv(tA, torch.from_numpy(x).to(dev), trans=trans)
        torch.cuda.synchronize()
        ref = ob.gemv(A, x, trans)
        assert y.dtype == torch.float32
        assert (np.abs(y.cpu().numpy() - ref) / _scale(A, x, trans)).max() <= 1e-5


@pytest.mark.parametrize("accu", [0, 1, 2])
@pytest.mark.parametrize("trans", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemv_fp16_levels(Bl, dev, shape, trans, accu):
    rows, cols = shape
    rng = np.random.default_rng(rows + 7 * cols + accu)
    A = rng.normal(0, 0.05, (rows, cols)).astype(np.float16)
    x = rng.normal(0, 0.05, rows if trans else cols).astype(np.float16)
    tA = _pitched(torch.from_numpy(A).to(dev), 8)
    y = Bl.gemv(tA, torch.from_numpy(x).to(dev), trans=trans, fp16_accu=accu)
    torch.cuda.synchronize()
    y32, y64, mag = ob.gemv(A, x, trans)
    got = y.cpu().numpy().astype(np.float64)
    scale = _scale(A, x, trans)
    assert y.dtype == (torch.float32 if accu == 0 else torch.float16)
    # fp16 results below 2^-14 are subnormal (absolute spacing 2^-24): allow half a step on top of the metric
    assert (np.abs(got - y64) <= 1e-2 * scale + (2.0 ** -25 if accu else 0.0)).all()
    if accu == 0:
        # fp32 arithmetic in another summation order: a few fp32 ulps of the summed magnitudes
        assert (np.abs(got - y64) <= 64 * 2.0 ** -24 * mag + 1e-30).all()
    elif accu == 1:
        # the fp32 value rounded once to fp16
        assert (np.abs(got - y64) <= 2.0 ** -11 * np.abs(y64) + 64 * 2.0 ** -24 * mag + 2.0 ** -25).all()


def test_gemv_without_workspace_gives_the_same_class_of_result(Bl, dev):
    """No scratch: the call falls back to one slice; same tolerance."""
    from decx_b200 import capi
    rng = np.random.default_rng(5)
    A = rng.uniform(-1, 1, (8, 40000)).astype(np.float32)
    x = rng.uniform(-1, 1, 40000).astype(np.float32)
    tA, tx = torch.from_numpy(A).to(dev), torch.from_numpy(x).to(dev)
    y = torch.empty(8, dtype=torch.float32, device=dev)
    assert capi.lib.decxb200_gemv_workspace_bytes(capi.FP32, 0, 0, 8, 40000) > 0
    capi.check(capi.lib.decxb200_gemv(capi.FP32, 0, 0, None, 8, 40000, tA.data_ptr(), 40000, tx.data_ptr(), y.data_ptr(), None, 0))
    torch.cuda.synchronize()
    assert (np.abs(y.cpu().numpy() - ob.gemv(A, x)) / _scale(A, x, False)).max() <= 1e-5


def test_gemv_is_deterministic(Bl, dev):
    rng = np.random.default_rng(6)
    A = torch.from_numpy(rng.uniform(-1, 1, (64, 30000)).astype(np.float32)).to(dev)
    x = torch.from_numpy(rng.uniform(-1, 1, 30000).astype(np.float32)).to(dev)
    y0 = Bl.gemv(A, x).clone()
    for _ in range(3):
        assert torch.equal(Bl.gemv(A, x), y0)


def test_gemv_argument_errors(Bl, dev):
    from decx_b200 import capi
    A = torch.zeros(4, 4, device=dev)
    assert capi.lib.decxb200_gemv(9, 0, 0, None, 4, 4, A.data_ptr(), 4, A.data_ptr(), A.data_ptr(), None, 0) == -1
    assert capi.lib.decxb200_gemv(capi.FP16, 3, 0, None, 4, 4, A.data_ptr(), 4, A.data_ptr(), A.data_ptr(), None, 0) == -1
    assert capi.lib.decxb200_gemv(capi.FP32, 0, 0, None, 4, 4, A.data_ptr(), 3, A.data_ptr(), A.data_ptr(), None, 0) == -1
    with pytest.raises(RuntimeError):
        Bl.gemv(torch.zeros(4, 4), torch.zeros(4))
