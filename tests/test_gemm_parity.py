"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bar (the path's contract): max_ij |D - D_ref| / (||A_i,:|| * ||B_:,j||) <= 1e-5 for fp32 and
complex-fp32 against an fp64 reference, <= 1e-2 for fp16 against an fp32-accumulating reference.
"""
import os

import numpy as np
import pytest

from oracle import binding as ob
from util import TOL, Guarded, make_inputs

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_cpu_gemm.npz")

DTYPES = [np.float32, np.float16, np.complex64]
# edge sizes of the reference's tiles and of this kernel's (64/128/256), the reference sample's
# ragged dims, and one-element extremes
SHAPES = [
    (1, 1, 1), (1, 7, 5), (7, 1, 3), (5, 3, 1), (8, 8, 8), (15, 17, 16), (16, 15, 17), (17, 16, 15),
    (63, 65, 64), (64, 63, 65), (65, 64, 63), (127, 129, 128), (128, 127, 129), (129, 128, 127),
    (255, 257, 256), (256, 255, 257), (257, 256, 255), (300, 520, 70), (513, 257, 33),
]


def _alpha_beta(dt):
    return (0.75 - 0.5j, -1.25 + 0.5j) if np.dtype(dt) == np.complex64 else (0.75, -1.25)


def _run(G, dev, A, B, C=None, alpha=None, beta=None, cta_group=0, poison=True):
    gA, gB = Guarded(torch, A, dev), Guarded(torch, B, dev)
    gC = Guarded(torch, C, dev) if C is not None else None
    gD = Guarded(torch, np.zeros((A.shape[0], B.shape[1]), dtype=A.dtype), dev, fill_logical=0)
    st = G.new_status(dev)
    G.gemm(gA.view, gB.view, gC.view if gC else None, alpha, beta, out=gD.view, status=st, cta_group=cta_group)
    torch.cuda.synchronize()
    assert int(st.item()) == 0, f"kernel status {int(st.item()):#x}"
    for g in (gA, gB, gD) + ((gC,) if gC else ()):
        g.check()
    return gD.view.cpu().numpy()


def _check(D, A, B, C=None, alpha=1.0, beta=0.0):
    ref = ob.gemm(A, B, C, alpha, beta)
    m = ob.metric(D, ref, A, B)
    assert m <= TOL[np.dtype(A.dtype).name], f"metric {m:.3e} for {A.dtype} {A.shape}x{B.shape}"
    return m


@pytest.fixture(scope="module")
def G():
    from decx_b200 import gemm
    assert torch.cuda.is_available()
    return gemm


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_plain_sweep(G, dev, dt, shape, cta_group):
    M, N, K = shape
    A, B, _ = make_inputs(dt, M, N, K, seed=M * 7 + N * 3 + K)
    _check(_run(G, dev, A, B, cta_group=cta_group), A, B)


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("shape", SHAPES[::2])
def test_fused_sweep(G, dev, dt, shape, cta_group):
    M, N, K = shape
    A, B, C = make_inputs(dt, M, N, K, seed=M + N + K, dist="normal", with_c=True)
    alpha, beta = _alpha_beta(dt)
    _check(_run(G, dev, A, B, C, alpha, beta, cta_group=cta_group), A, B, C, alpha, beta)


@pytest.mark.parametrize("name", ["f32_64", "f32_ragged", "f32_192", "c64_64", "c64_128x64x46", "c64_128"])
def test_against_reference_cpu_gemm_outputs(G, dev, name):
    """Golden vectors produced by the reference's own de::blas::cpu::GEMM (tests/golden/)."""
    z = np.load(GOLD)
    A, B, Dref = z[name + "_A"], z[name + "_B"], z[name + "_D"]
    D = _run(G, dev, A, B)
    assert ob.metric(D, Dref, A, B) <= 1e-5


def test_reference_sample_known_answer(G, dev):
    """samples/Matrix_Multiplication/MatMul.cpp:64-140: complex fused GEMM, W=1013 H=1077 L=1005,
    A = (j, 0), B = (i, 0), C = (1e6, 1e6): every element is (sum i^2 + 1e6, 1e6).  All inputs are
    positive, so rounding errors add up instead of cancelling: a stress of the 3xTF32 split."""
    W, H, L = 1013, 1077, 1005
    A = np.tile(np.arange(L, dtype=np.float32), (H, 1)).astype(np.complex64)
    B = np.tile(np.arange(L, dtype=np.float32)[:, None], (1, W)).astype(np.complex64)
    C = np.full((H, W), 1e6 + 1e6j, dtype=np.complex64)
    D = _run(G, dev, A, B, C, 1.0, 1.0)
    expect = sum(i * i for i in range(L)) + 1e6
    assert np.abs(D.real.astype(np.float64) - expect).max() / expect < 2e-6
    assert np.abs(D.imag.astype(np.float64) - 1e6).max() / expect < 2e-6
    _check(D, A, B, C, 1.0, 1.0)


def test_k_equal_one_exposes_per_product_error(G, dev):
    """With K = 1 the metric is the relative error of a single product: 1xTF32 would give 5e-4."""
    rng = np.random.default_rng(3)
    A = rng.uniform(-1, 1, (300, 1)).astype(np.float32)
    B = rng.uniform(-1, 1, (1, 500)).astype(np.float32)
    m = _check(_run(G, dev, A, B), A, B)
    assert m < 2e-6


def test_baseline_cfg3_fused_ragged_full(G, dev):
    """fp32 D = A.B + C, M=4099 N=3001 K=2053, N(0,1) inputs, alpha = beta = 1; whole matrix checked."""
    A, B, C = make_inputs(np.float32, 4099, 3001, 2053, seed=2, dist="normal", with_c=True)
    _check(_run(G, dev, A, B, C, 1.0, 1.0), A, B, C, 1.0, 1.0)


def _rows_check(D_rows, A_rows, B, tol):
    ref = ob.gemm(A_rows, B)
    m = ob.metric(D_rows, ref, A_rows, B)
    assert m <= tol, f"metric {m:.3e}"


def test_baseline_cfg2_fp32_8192_sampled_rows(G, dev):
    """fp32 8192^3, U[-1,1]: 48 sampled rows (tile edges included) against the fp64 oracle."""
    A, B, _ = make_inputs(np.float32, 8192, 8192, 8192, seed=1)
    tA, tB = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)
    st = G.new_status(dev)
    D = G.gemm(tA, tB, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    rows = sorted(set([0, 1, 127, 128, 255, 256, 4095, 4096, 8191] + list(np.random.default_rng(0).integers(0, 8192, 39))))
    _rows_check(D[rows].cpu().numpy(), A[rows], B, 1e-5)
    # the same rows as their own problem give the same bits (K order does not depend on M)
    D2 = G.gemm(tA[4096:4352].contiguous(), tB)
    torch.cuda.synchronize()
    assert torch.equal(D2, D[4096:4352])


def test_baseline_cfg4_cplxf_4096_sampled_rows(G, dev):
    A, B, _ = make_inputs(np.complex64, 4096, 4096, 4096, seed=3)
    tA, tB = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)
    D = G.gemm(tA, tB)
    torch.cuda.synchronize()
    rows = sorted(set([0, 127, 128, 2047, 2048, 4095] + list(np.random.default_rng(1).integers(0, 4096, 26))))
    _rows_check(D[rows].cpu().numpy(), A[rows], B, 1e-5)


def test_baseline_cfg5_shape_fp16_properties(G, dev):
    """fp16 with N = K = 16384 as in the sharded configuration (8192 of its 65536 rows = one of
    eight shards): sampled rows against the oracle, exact identity and power-of-two scaling."""
    M, N, K = 8192, 16384, 16384
    g = torch.Generator(device=dev).manual_seed(4)
    tA = (torch.randn(M, K, device=dev, generator=g) * 0.02).half()
    tB = (torch.randn(K, N, device=dev, generator=g) * 0.02).half()
    D = G.gemm(tA, tB)
    torch.cuda.synchronize()
    rows = [0, 127, 128, 255, 256, 4095, 8191] + list(np.random.default_rng(2).integers(0, M, 9))
    A_rows, Bh = tA[rows].cpu().numpy(), tB.cpu().numpy()
    _rows_check(D[rows].cpu().numpy(), A_rows, Bh, 1e-2)
    # alpha = 2 doubles the fp32 accumulator exactly, so every fp16 result that is a normal number
    # doubles exactly (subnormal results round on a fixed grid and are left out; nothing overflows)
    D2 = G.gemm(tA, tB, alpha=2.0)
    torch.cuda.synchronize()
    normal = D.float().abs() >= 2.0 ** -13
    assert normal.float().mean() > 0.99
    assert torch.equal(D2.float()[normal], (D.float() * 2)[normal])
    # A . I == A bit for bit (one exact product per output, fp32 accumulate, exact fp16 store)
    eye = torch.eye(K, dtype=torch.float16, device=dev)
    assert torch.equal(G.gemm(tA, eye), tA)


def test_beta_zero_ignores_c_and_alpha_scales(G, dev):
    A, B, _ = make_inputs(np.float32, 130, 70, 40, seed=5)
    C = np.full((130, 70), np.nan, dtype=np.float32)
    D = _run(G, dev, A, B, C, 2.0, 0.0)
    _check(D, A, B, None, 2.0, 0.0)


def test_zero_inputs_give_exact_zero(G, dev):
    for dt in DTYPES:
        A = np.zeros((140, 90), dtype=dt)
        B = make_inputs(dt, 90, 75, 90, seed=1)[1][:90, :75]
        D = _run(G, dev, A, np.ascontiguousarray(B))
        assert not D.any()


def test_argument_errors_through_the_c_abi(G, dev):
    from decx_b200 import capi
    A = torch.zeros(64, 72, dtype=torch.float16, device=dev)
    with pytest.raises(capi.DecxB200Error) as e:
        G.gemm(A[:, :71][:, 1:], torch.zeros(70, 64, dtype=torch.float16, device=dev))   # misaligned base
    assert e.value.code == -2
    with pytest.raises(capi.DecxB200Error) as e:
        G.gemm(torch.zeros(64, 70, dtype=torch.float16, device=dev)[:, :64],
               torch.zeros(64, 64, dtype=torch.float16, device=dev))                       # pitch of 70 halves
    assert e.value.code == -2
    a32 = torch.zeros(64, 64, device=dev)
    code = capi.lib.decxb200_gemm(capi.FP32, None, 64, 64, 64, a32.data_ptr(), 64, a32.data_ptr(), 64, None, 0,
                                  a32.data_ptr(), 64, None, None, None, 0, None)
    assert code == -3                                                                      # no workspace
    with pytest.raises(RuntimeError):
        G.gemm(torch.zeros(4, 4), torch.zeros(4, 4))                                       # CPU tensors: no fallback


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("pinned", [True, False])
def test_host_pointer_entry_point(G, dev, dt, pinned):
    """decxb200_gemm_host: several row blocks (M > 2048), pitched host matrices, fused form."""
    M, N, K = 5000, 520, 300
    A, B, C = make_inputs(dt, M, N, K, seed=9, dist="normal", with_c=True)
    alpha, beta = _alpha_beta(dt)
    hp = lambda x: torch.from_numpy(np.pad(x, ((0, 0), (0, 5))))[:, : x.shape[1]]        # host pitch > width
    tA, tB, tC = hp(A), hp(B), hp(C)
    if pinned:
        tA, tB, tC = (torch.from_numpy(np.pad(x, ((0, 0), (0, 5)))).pin_memory()[:, : x.shape[1]] for x in (A, B, C))
    st = G.new_status(dev)
    out = torch.full((M, N + 3), complex("nan+nanj") if tA.is_complex() else float("nan"), dtype=tA.dtype)
    if pinned:
        out = out.pin_memory()
    G.gemm_host(tA, tB, tC, alpha, beta, out=out[:, :N], status=st, device=dev)
    assert int(st.item()) == 0
    o = torch.view_as_real(out) if out.is_complex() else out
    assert torch.isnan(o[:, N:]).all()
    _check(out[:, :N].numpy(), A, B, C, alpha, beta)
    # same numbers as the device-pointer entry point, bit for bit
    gA, gB, gC = (Guarded(torch, x, dev) for x in (A, B, C))
    D = G.gemm(gA.view, gB.view, gC.view, alpha, beta)
    torch.cuda.synchronize()
    assert torch.equal(D.cpu(), out[:, :N])


def test_host_pointer_fp16_large_b_goes_up_in_column_panels(G, dev):
    """fp16 with a B of 64 MiB and no C: the first row block is multiplied panel by panel of B while B is still
    being uploaded (ragged M, N not a multiple of the panel width, pitched host matrices); same bits as the
    device-pointer entry point, and the oracle agrees on sampled rows."""
    M, N, K = 2300, 4104, 8192
    A, B, _ = make_inputs(np.float16, M, N, K, seed=21, dist="small")
    hp = lambda x: torch.from_numpy(np.pad(x, ((0, 0), (0, 8)))).pin_memory()[:, : x.shape[1]]
    tA, tB = hp(A), hp(B)
    st = G.new_status(dev)
    out = torch.full((M, N + 8), float("nan"), dtype=torch.float16).pin_memory()
    G.gemm_host(tA, tB, out=out[:, :N], status=st, device=dev)
    assert int(st.item()) == 0
    assert torch.isnan(out[:, N:]).all()
    D = G.gemm(torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev))
    torch.cuda.synchronize()
    assert torch.equal(D.cpu(), out[:, :N])
    rows = [0, 1023, 1024, 2047, 2048, M - 1]
    ref = ob.gemm(A[rows], B)
    assert ob.metric(out[rows, :N].numpy(), ref, A[rows], B) <= TOL["float16"]


def test_huge_finite_fp32_inputs_do_not_turn_into_nan(G, dev):
    """Values next to FLT_MAX: rounding them up to tf32 would overflow; the split keeps them finite."""
    rng = np.random.default_rng(12)
    A = rng.uniform(-1, 1, (70, 40)).astype(np.float32)
    B = rng.uniform(-1e-3, 1e-3, (40, 50)).astype(np.float32)
    fmax = np.finfo(np.float32).max
    A[3, 5], A[10, 0], A[69, 39] = fmax, -fmax, 3.4e38
    D = _run(G, dev, A, B)
    assert np.isfinite(D).all()
    _check(D, A, B)
