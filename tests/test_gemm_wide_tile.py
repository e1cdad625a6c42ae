"""GPU parity tests of the 256 x 512 pair tile (two TMEM accumulators per tile, `gemm_tcgen05_kernel<0,2,2>`).

This is the kernel the large fp16 problems and the row-sharded multi-GPU path run.  The library picks it by a
cost model only for long K and many tiles, so the tests force it (DECXB200_TILE_256x512) on small ragged
shapes: M not a multiple of 256, N not a multiple of 512 / 256 / 64 / 8, pitched and unpitched D, with and
without panel gating.  Everything is compared with the CPU oracle by the path's metric (fp16: <= 1e-2).
"""
import time

import numpy as np
import pytest

from oracle import binding as ob
from util import TOL, Guarded, make_inputs

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

WIDE = 3     # DECXB200_TILE_256x512

# (M, N, K): ragged against 256 rows and 512 / 256 / 64 columns; K from one k-block to long, ragged too
SHAPES = [
    (256, 512, 2048), (257, 2000, 2053), (1300, 2104, 2048), (512, 1992, 2304), (300, 520, 70), (129, 513, 64),
    (1, 1, 1), (255, 511, 4099), (770, 1031, 2050),
]


@pytest.fixture(scope="module")
def G():
    from decx_b200 import gemm
    assert torch.cuda.is_available()
    return gemm


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _variant():
    from decx_b200 import capi
    return capi.lib.decxb200_last_kernel_variant()


def _metric(D, A, B, C=None, alpha=1.0, beta=0.0):
    ref = ob.gemm(A, B, C, alpha, beta)
    return ob.metric(D, ref, A, B)


@pytest.mark.parametrize("shape", SHAPES)
def test_wide_tile_plain_ragged(G, dev, shape):
    M, N, K = shape
    A, B, _ = make_inputs(np.float16, M, N, K, seed=M + 3 * N + 7 * K, dist="small")
    gA, gB = Guarded(torch, A, dev), Guarded(torch, B, dev)
    gD = Guarded(torch, np.zeros((M, N), np.float16), dev, fill_logical=0)
    st = G.new_status(dev)
    G.gemm(gA.view, gB.view, out=gD.view, status=st, cta_group=WIDE)
    torch.cuda.synchronize()
    assert _variant() == 22
    assert int(st.item()) == 0
    for g in (gA, gB, gD):
        g.check()
    assert _metric(gD.view.cpu().numpy(), A, B) <= TOL["float16"]


@pytest.mark.parametrize("shape", [(257, 2000, 2053), (1300, 2104, 2048), (300, 520, 70)])
def test_wide_tile_fused_ragged(G, dev, shape):
    M, N, K = shape
    A, B, C = make_inputs(np.float16, M, N, K, seed=5 + M, dist="small", with_c=True)
    gA, gB, gC = (Guarded(torch, x, dev) for x in (A, B, C))
    gD = Guarded(torch, np.zeros((M, N), np.float16), dev, fill_logical=0)
    st = G.new_status(dev)
    G.gemm(gA.view, gB.view, gC.view, 0.75, -1.25, out=gD.view, status=st, cta_group=WIDE)
    torch.cuda.synchronize()
    assert _variant() == 22 and int(st.item()) == 0
    for g in (gA, gB, gC, gD):
        g.check()
    assert _metric(gD.view.cpu().numpy(), A, B, C, 0.75, -1.25) <= TOL["float16"]


@pytest.mark.parametrize("shape", [(300, 2001, 2048), (513, 1027, 128)])
def test_wide_tile_unpitched_d_uses_predicated_stores(G, dev, shape):
    """D with a row pitch that is not a multiple of 16 bytes: no TMA store, per-thread predicated stores."""
    M, N, K = shape
    A, B, _ = make_inputs(np.float16, M, N, K, seed=2, dist="small")
    gA, gB = Guarded(torch, A, dev), Guarded(torch, B, dev)
    D = torch.full((M + 2, N), float("nan"), dtype=torch.float16, device=dev)
    st = G.new_status(dev)
    G.gemm(gA.view, gB.view, out=D[1:M + 1], status=st, cta_group=WIDE)
    torch.cuda.synchronize()
    assert _variant() == 22 and int(st.item()) == 0
    assert torch.isnan(D[0]).all() and torch.isnan(D[M + 1]).all()
    assert _metric(D[1:M + 1].cpu().numpy(), A, B) <= TOL["float16"]


def test_wide_tile_equals_plain_pair_tile_bitwise(G, dev):
    """Same K order and the same fp32 accumulation per output element: the two tile shapes agree bit for bit."""
    A, B, _ = make_inputs(np.float16, 1300, 2104, 2304, seed=9, dist="small")
    tA, tB = Guarded(torch, A, dev).view, Guarded(torch, B, dev).view
    D2 = G.gemm(tA, tB, cta_group=2)
    D3 = G.gemm(tA, tB, cta_group=WIDE)
    torch.cuda.synchronize()
    assert torch.equal(D2, D3)


# ------------------------------------------------------------------ panel gating on the wide tile
PANEL_CASES = [
    # (M, N, K, panel ends)
    (1300, 2104, 2048, [512, 1536, 2104]),
    (257, 2000, 2053, [1024, 2000]),
    (512, 4096, 2048, [512, 1024, 2048, 2560, 3072, 3584, 4096]),
    (770, 1992, 2304, [1992]),
]


@pytest.mark.parametrize("case", PANEL_CASES)
def test_wide_tile_panels_flags_preset(G, dev, case):
    M, N, K, ends = case
    A, B, _ = make_inputs(np.float16, M, N, K, seed=N, dist="small")
    gA, gB = Guarded(torch, A, dev), Guarded(torch, B, dev)
    gD = Guarded(torch, np.zeros((M, N), np.float16), dev, fill_logical=0)
    st = G.new_status(dev)
    flags = torch.full((16,), 3, dtype=torch.int32, device=dev)
    G.gemm_fp16_panels(gA.view, gB.view, gD.view, ends, flags, 3, status=st, tile=WIDE)
    torch.cuda.synchronize()
    assert _variant() == 22 and int(st.item()) == 0
    for g in (gA, gB, gD):
        g.check()
    assert _metric(gD.view.cpu().numpy(), A, B) <= TOL["float16"]


@pytest.mark.parametrize("case", PANEL_CASES[:3])
def test_wide_tile_panels_delivered_late_by_a_side_stream(G, dev, case):
    """The GEMM is launched over an all-zero B; a side stream then copies the panels in, LAST panel first,
    flagging each one.  The loader must wait for every panel's flag and must see the delivered data."""
    M, N, K, ends = case
    A, B, _ = make_inputs(np.float16, M, N, K, seed=N + 1, dist="small")
    gA, gB = Guarded(torch, A, dev), Guarded(torch, B, dev)
    gBdst = Guarded(torch, np.zeros_like(B), dev)
    gD = Guarded(torch, np.zeros((M, N), np.float16), dev, fill_logical=0)
    st = G.new_status(dev)
    flags = torch.zeros(16, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(dev)
    G.gemm_fp16_panels(gA.view, gBdst.view, gD.view, ends, flags, 1, status=st, tile=WIDE)
    time.sleep(0.02)
    pitch = gB.pitch * 2
    starts = [0] + ends[:-1]
    with torch.cuda.stream(side):
        for i in reversed(range(len(ends))):
            lo, hi = starts[i], ends[i]
            G.copy2d(gBdst.view.data_ptr() + 2 * lo, pitch, gB.view.data_ptr() + 2 * lo, pitch, 2 * (hi - lo), K, side)
            G.write_flag(flags, i, 1, side)
            time.sleep(0.005)
    torch.cuda.synchronize()
    assert _variant() == 22 and int(st.item()) == 0
    gD.check()
    assert _metric(gD.view.cpu().numpy(), A, B) <= TOL["float16"]
    ref = G.gemm(gA.view, gB.view, cta_group=WIDE)
    torch.cuda.synchronize()
    assert torch.equal(ref, gD.view)


def test_forced_wide_tile_rejects_panel_ends_off_the_tile_grid(G, dev):
    from decx_b200 import capi
    A = torch.zeros(256, 64, dtype=torch.float16, device=dev)
    B = torch.zeros(64, 1024, dtype=torch.float16, device=dev)
    out = torch.empty(256, 1024, dtype=torch.float16, device=dev)
    flags = torch.ones(16, dtype=torch.int32, device=dev)
    with pytest.raises(capi.DecxB200Error) as e:
        G.gemm_fp16_panels(A, B, out, [256, 1024], flags, 1, tile=WIDE)
    assert e.value.code == -1
