"""GPU tests of the GEMM with in-kernel fetch of B (`decxb200_gemm_fp16_fetch`) on ONE GPU.

The courier warps copy pieces of B from "other GPUs" into the local replica while the tiles run.  Here the
sources are other buffers of the same GPU, which exercises everything but the NVLink hop: the job walk, the
batch arithmetic on ragged pieces, the per-panel counts, the ready flags the loader waits on, the publish flags,
gates opened late by a side stream (standing in for another GPU's progress), and wait-only jobs.  The result is
compared with the CPU oracle by the path's metric and bit for bit with the plain kernel.
"""
import time

import numpy as np
import pytest

from oracle import binding as ob
from util import TOL, Guarded, make_inputs

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
WIDE = 3


@pytest.fixture(scope="module")
def G():
    from decx_b200 import gemm
    return gemm


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _jobs(capi, src_ptrs, gates, K, ends, pieces, me):
    """Job list of 'rank' `me` among len(pieces) holders: piece `me` comes from the owner's B (src_ptrs[-1],
    no gate, published), the others from their holders' copies, gated on gates[holder] + 4*panel."""
    jobs, c0 = [], 0
    for p, c1 in enumerate(ends):
        order = [me] + [(me + d) % len(pieces) for d in range(1, len(pieces))]
        for h in order:
            r0, nr = pieces[h]
            if nr == 0:
                continue
            own = h == me
            jobs.append(capi.fetch_job(src_ptrs[-1] if own else src_ptrs[h], None if own else gates[h] + 4 * p,
                                      r0, nr, c0, c1 - c0, p, 1 if own else 0))
        c0 = c1
    return jobs


CASES = [
    # M, N, K, panel ends, row pieces [(row0, rows)], tile
    (512, 1024, 256, [512, 1024], [(0, 128), (128, 128)], 0),
    (1300, 2104, 2048, [512, 1536, 2104], [(0, 704), (704, 640), (1344, 704)], WIDE),
    (257, 2000, 2053, [1024, 2000], [(0, 1000), (1000, 1053)], WIDE),
    (768, 4096, 512, [512, 1024, 1536, 2048, 2560, 3072, 3584, 4096], [(0, 73), (73, 73), (146, 73), (219, 73), (292, 73), (365, 73), (438, 74)], WIDE),
    (300, 520, 70, [520], [(0, 70)], 0),
]


@pytest.mark.parametrize("staged", [False, True])
@pytest.mark.parametrize("case", CASES)
def test_fetch_from_local_stand_ins_gates_preset(G, dev, case, staged):
    """staged: D leaves through the per-CTA ring and the couriers' 16-byte stores (what a rank does whose D rows live
    in another GPU's memory) instead of the epilogue's own TMA stores; the guard rows and columns around D show
    that the couriers clip at M and N."""
    from decx_b200 import capi
    M, N, K, ends, pieces, tile = case
    d_stage = torch.empty(capi.lib.decxb200_fetch_d_stage_bytes(), dtype=torch.uint8, device=dev) if staged else None
    A, B, _ = make_inputs(np.float16, M, N, K, seed=K + N, dist="small")
    gA, gB = Guarded(torch, A, dev), Guarded(torch, B, dev)
    holders = [Guarded(torch, B, dev) for _ in pieces]                 # what the other "ranks" hold
    gRep = Guarded(torch, np.zeros_like(B), dev)                       # this rank's replica, empty
    gD = Guarded(torch, np.zeros((M, N), np.float16), dev, fill_logical=0)
    st = G.new_status(dev)
    ready = torch.zeros(16, dtype=torch.int32, device=dev)
    pub = torch.zeros(16, dtype=torch.int32, device=dev)
    gates = torch.full((len(pieces), 16), 9, dtype=torch.int32, device=dev)
    src = [h.view.data_ptr() for h in holders] + [gB.view.data_ptr()]
    jobs = _jobs(capi, src, [gates[i].data_ptr() for i in range(len(pieces))], K, ends, pieces, me=0)
    scratch = torch.empty(capi.lib.decxb200_fetch_scratch_bytes(len(jobs)), dtype=torch.uint8, device=dev)
    G.gemm_fp16_fetch(gA.view, gRep.view, gD.view.data_ptr(), gD.pitch, ends, ready, pub, 9, jobs, scratch,
                      status=st, tile=tile, d_stage=d_stage)
    torch.cuda.synchronize()
    assert capi.lib.decxb200_last_kernel_variant() in (1021, 1022)
    assert int(st.item()) == 0
    for g in (gA, gB, gRep, gD):
        g.check()
    assert torch.equal(gRep.view, gB.view)                             # the replica is complete and exact
    assert (ready[:len(ends)] == 9).all() and (pub[:len(ends)] == 9).all()
    ref = ob.gemm(A, B)
    assert ob.metric(gD.view.cpu().numpy(), ref, A, B) <= TOL["float16"]
    plain = G.gemm(gA.view, gB.view, cta_group=WIDE if tile == WIDE else 2)
    torch.cuda.synchronize()
    assert torch.equal(plain, gD.view)


def test_fetch_gates_opened_late_and_wait_only_piece(G, dev):
    """Holder 1's pieces only become readable when a side stream (standing in for that GPU's progress) has
    written them and raised their flags; holder 2's piece is delivered into the replica by a copy engine and the
    job only waits for its flag (rows == 0)."""
    from decx_b200 import capi
    M, N, K, ends = 1024, 2048, 2048, [512, 1024, 2048]
    A, B, _ = make_inputs(np.float16, M, N, K, seed=77, dist="small")
    gA, gB = Guarded(torch, A, dev), Guarded(torch, B, dev)
    h1 = Guarded(torch, np.zeros_like(B), dev)                          # fills up late
    gRep = Guarded(torch, np.zeros_like(B), dev)
    gD = Guarded(torch, np.zeros((M, N), np.float16), dev, fill_logical=0)
    st = G.new_status(dev)
    ready, pub = torch.zeros(16, dtype=torch.int32, device=dev), torch.zeros(16, dtype=torch.int32, device=dev)
    gate1, gate2 = torch.zeros(16, dtype=torch.int32, device=dev), torch.zeros(16, dtype=torch.int32, device=dev)
    rows = [(0, 700), (700, 648), (1348, 700)]
    jobs, c0 = [], 0
    for p, c1 in enumerate(ends):
        jobs.append(capi.fetch_job(gB.view.data_ptr(), None, rows[0][0], rows[0][1], c0, c1 - c0, p, 1))
        jobs.append(capi.fetch_job(h1.view.data_ptr(), gate1.data_ptr() + 4 * p, rows[1][0], rows[1][1], c0, c1 - c0, p, 0))
        jobs.append(capi.fetch_job(None, gate2.data_ptr() + 4 * p, rows[2][0], 0, c0, c1 - c0, p, 0))
        c0 = c1
    scratch = torch.empty(capi.lib.decxb200_fetch_scratch_bytes(len(jobs)), dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(dev)
    G.gemm_fp16_fetch(gA.view, gRep.view, gD.view.data_ptr(), gD.pitch, ends, ready, pub, 2, jobs, scratch,
                      status=st, tile=WIDE)
    time.sleep(0.02)
    pitch = gB.pitch * 2
    with torch.cuda.stream(side):
        c0 = 0
        for p, c1 in enumerate(ends):
            for dst, gate, (r0, nr) in ((h1, gate1, rows[1]), (gRep, gate2, rows[2])):
                off = r0 * pitch + 2 * c0
                G.copy2d(dst.view.data_ptr() + off, pitch, gB.view.data_ptr() + off, pitch, 2 * (c1 - c0), nr, side)
                G.write_flag(gate, p, 2, side)
            time.sleep(0.005)
            c0 = c1
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    gRep.check()
    gD.check()
    assert torch.equal(gRep.view, gB.view)
    assert (ready[:3] == 2).all() and (pub[:3] == 2).all()
    plain = G.gemm(gA.view, gB.view, cta_group=WIDE)
    torch.cuda.synchronize()
    assert torch.equal(plain, gD.view)
    assert ob.metric(gD.view.cpu().numpy(), ob.gemm(A, B), A, B) <= TOL["float16"]


def test_fetch_argument_errors(G, dev):
    from decx_b200 import capi
    A = torch.zeros(256, 64, dtype=torch.float16, device=dev)
    B = torch.zeros(64, 1024, dtype=torch.float16, device=dev)
    D = torch.zeros(256, 1024, dtype=torch.float16, device=dev)
    flags = torch.zeros(32, dtype=torch.int32, device=dev)
    scratch = torch.empty(4096, dtype=torch.uint8, device=dev)
    ok = capi.fetch_job(B.data_ptr(), None, 0, 64, 0, 512, 0, 1)

    def call(jobs, ends=(512, 1024)):
        G.gemm_fp16_fetch(A, B, D.data_ptr(), 1024, list(ends), flags[:16], flags[16:], 1, jobs, scratch)

    for bad in ([ok],                                                            # panel 1 has no job
                [ok, capi.fetch_job(B.data_ptr(), None, 0, 64, 256, 512, 1, 0)],  # columns outside the panel
                [ok, capi.fetch_job(B.data_ptr(), None, 32, 64, 512, 512, 1, 0)], # rows beyond K
                [ok, capi.fetch_job(None, None, 0, 0, 512, 512, 1, 0)]):          # wait-only piece without a gate
        with pytest.raises(capi.DecxB200Error) as e:
            call(bad)
        assert e.value.code == -1


def test_push_jobs_fill_another_replica_and_raise_its_flags(G, dev):
    """The owner's side of the scatter: while it multiplies with the B it already holds (no gating), its couriers
    store row pieces of every panel into two other replicas (other GPUs' memory in the real run) and raise the
    targets' flags when a piece is complete."""
    from decx_b200 import capi
    M, N, K, ends = 770, 2104, 520, [512, 1536, 2104]
    A, B, _ = make_inputs(np.float16, M, N, K, seed=31, dist="small")
    gA, gB = Guarded(torch, A, dev), Guarded(torch, B, dev)
    targets = [Guarded(torch, np.zeros_like(B), dev) for _ in range(2)]
    tflags = torch.zeros((2, 16), dtype=torch.int32, device=dev)
    gD = Guarded(torch, np.zeros((M, N), np.float16), dev, fill_logical=0)
    st = G.new_status(dev)
    pieces = [(0, 272), (272, 248)]
    jobs, c0 = [], 0
    for p, c1 in enumerate(ends):
        for k in range(2):
            q = (p + k) % 2
            jobs.append(capi.fetch_job(gB.view.data_ptr(), None, pieces[q][0], pieces[q][1], c0, c1 - c0, p, 0,
                                       dst=targets[q].view.data_ptr(), notify=tflags[q].data_ptr() + 4 * p))
        c0 = c1
    scratch = torch.empty(capi.lib.decxb200_fetch_scratch_bytes(len(jobs)), dtype=torch.uint8, device=dev)
    G.gemm_fp16_fetch(gA.view, gB.view, gD.view.data_ptr(), gD.pitch, ends, None, None, 4, jobs, scratch, status=st, tile=WIDE)
    torch.cuda.synchronize()
    assert capi.lib.decxb200_last_kernel_variant() == 1022 and int(st.item()) == 0
    for q, t in enumerate(targets):
        t.check()
        r0, nr = pieces[q]
        assert torch.equal(t.view[r0:r0 + nr], gB.view[r0:r0 + nr])          # its piece, every panel
        other = pieces[1 - q]
        assert not t.view[other[0]:other[0] + other[1]].any()                # and nothing else
        assert (tflags[q, :3] == 4).all() and not tflags[q, 3:].any()
    gB.check()
    gD.check()
    plain = G.gemm(gA.view, gB.view, cta_group=WIDE)
    torch.cuda.synchronize()
    assert torch.equal(plain, gD.view)
    # push jobs may not publish, pull jobs may not notify
    bad = capi.fetch_job(gB.view.data_ptr(), None, 0, 16, 0, 512, 0, 1, dst=targets[0].view.data_ptr())
    with pytest.raises(capi.DecxB200Error):
        G.gemm_fp16_fetch(gA.view, gB.view, gD.view.data_ptr(), gD.pitch, ends, None, None, 5, [bad], scratch)
