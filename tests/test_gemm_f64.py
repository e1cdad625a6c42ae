"""GPU parity tests of the fp64 and complex-fp64 GEMM (warp-level DMMA kernel) through the C ABI.

Bar: max |D - D_ref| / (||A_i|| ||B_j||) <= 1e-13 against the long-double oracle (fp64 rounding is 1.1e-16 per
operation; the observed metric is a few 1e-16)."""
import numpy as np
import pytest

from oracle import binding as ob
from util import Guarded, make_inputs

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
TOL64 = 1e-13

SHAPES = [(1, 1, 1), (7, 5, 3), (8, 8, 4), (17, 16, 15), (64, 63, 65), (127, 129, 128), (129, 128, 127),
          (255, 257, 31), (300, 520, 70), (513, 131, 33), (128, 128, 1000)]


@pytest.fixture(scope="module")
def G():
    from decx_b200 import gemm
    return gemm


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _run(G, dev, A, B, C=None, alpha=None, beta=None):
    gA, gB = Guarded(torch, A, dev), Guarded(torch, B, dev)
    gC = Guarded(torch, C, dev) if C is not None else None
    gD = Guarded(torch, np.zeros((A.shape[0], B.shape[1]), dtype=A.dtype), dev, fill_logical=0)
    G.gemm(gA.view, gB.view, gC.view if gC else None, alpha, beta, out=gD.view)
    torch.cuda.synchronize()
    for g in (gA, gB, gD) + ((gC,) if gC else ()):
        g.check()
    return gD.view.cpu().numpy()


@pytest.mark.parametrize("dt", [np.float64, np.complex128])
@pytest.mark.parametrize("shape", SHAPES)
def test_plain_sweep(G, dev, dt, shape):
    M, N, K = shape
    A, B, _ = make_inputs(dt, M, N, K, seed=M + 2 * N + 3 * K)
    D = _run(G, dev, A, B)
    assert ob.metric(D, ob.gemm(A, B), A, B) <= TOL64


@pytest.mark.parametrize("dt", [np.float64, np.complex128])
@pytest.mark.parametrize("shape", SHAPES[::2])
def test_fused_sweep(G, dev, dt, shape):
    M, N, K = shape
    A, B, C = make_inputs(dt, M, N, K, seed=M + N + K, dist="normal", with_c=True)
    alpha, beta = (0.75 - 0.5j, -1.25 + 0.5j) if dt == np.complex128 else (0.75, -1.25)
    D = _run(G, dev, A, B, C, alpha, beta)
    assert ob.metric(D, ob.gemm(A, B, C, alpha, beta), A, B) <= TOL64


def test_unaligned_pitch_uses_8_byte_copies(G, dev):
    """Odd row pitch: the 16-byte cp.async form is illegal, the kernel switches to 8-byte copies."""
    A, B, _ = make_inputs(np.float64, 130, 71, 45, seed=4)
    tA = torch.from_numpy(np.pad(A, ((0, 0), (0, 2)))).to(dev)[:, :45]          # pitch 47
    tB = torch.from_numpy(np.pad(B, ((0, 0), (0, 4)))).to(dev)[:, :71]          # pitch 75
    out = torch.zeros((130, 73), dtype=torch.float64, device=dev)[:, :71]
    G.gemm(tA, tB, out=out)
    torch.cuda.synchronize()
    assert ob.metric(out.cpu().numpy(), ob.gemm(A, B), A, B) <= TOL64


def test_fp64_keeps_what_fp32_loses(G, dev):
    """1 + 2^-40 style operands: the products differ from 1 far below fp32 resolution."""
    K = 64
    A = np.full((16, K), 1.0 + 2.0 ** -40)
    B = np.full((K, 24), 1.0 - 2.0 ** -41)
    D = _run(G, dev, A, B)
    exact = K * (1.0 + 2.0 ** -40) * (1.0 - 2.0 ** -41)
    assert np.abs(D - exact).max() <= 4 * K * 2.0 ** -53


def test_large_sampled_rows(G, dev):
    M = N = K = 2048
    A, B, _ = make_inputs(np.float64, M, N, K, seed=8)
    tA, tB = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)
    D = G.gemm(tA, tB)
    torch.cuda.synchronize()
    rows = [0, 63, 64, 127, 128, 1023, 2047]
    assert ob.metric(D[rows].cpu().numpy(), ob.gemm(A[rows], B), A[rows], B) <= TOL64
    Ac, Bc, _ = make_inputs(np.complex128, 1024, 1024, 1024, seed=9)
    Dc = G.gemm(torch.from_numpy(Ac).to(dev), torch.from_numpy(Bc).to(dev))
    torch.cuda.synchronize()
    rows = [0, 127, 128, 1023]
    assert ob.metric(Dc[rows].cpu().numpy(), ob.gemm(Ac[rows], Bc), Ac[rows], Bc) <= TOL64


def test_host_pointer_entry_point_fp64(G, dev):
    for dt in (np.float64, np.complex128):
        M, N, K = 2500, 200, 130
        A, B, C = make_inputs(dt, M, N, K, seed=10, dist="normal", with_c=True)
        alpha, beta = (0.5 - 0.25j, 1.0 + 0.5j) if dt == np.complex128 else (0.5, 1.0)
        out = G.gemm_host(torch.from_numpy(A), torch.from_numpy(B), torch.from_numpy(C), alpha, beta, device=dev)
        assert ob.metric(out.numpy(), ob.gemm(A, B, C, alpha, beta), A, B) <= TOL64
