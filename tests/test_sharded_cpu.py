"""CPU tests of the sharded GEMM's host logic: partition rules, and the whole broadcast /
multiply / gather schedule across two gloo ranks with an injected host GEMM."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from decx_b200.sharded import ShardedGemm, panel_plan, row_ranges  # noqa: E402


def test_row_ranges_cover_and_align():
    for M in (1, 255, 256, 257, 4099, 65536):
        for w in (1, 2, 3, 4, 8):
            rr = row_ranges(M, w)
            assert len(rr) == w and sum(n for _, n in rr) == M
            pos = 0
            for start, n in rr:
                if n:
                    assert start == pos and start % 256 == 0
                    pos += n
    assert row_ranges(65536, 8) == [(i * 8192, 8192) for i in range(8)]
    assert row_ranges(300, 4) == [(0, 256), (256, 44), (300, 0), (300, 0)]
    # a lighter share for one rank: its blocks go to the others, everything still covered in order
    rr = row_ranges(65536, 8, lighter=(0, 2))
    assert rr[0] == (0, 30 * 256) and sum(n for _, n in rr) == 65536 and sorted(n // 256 for _, n in rr) == [30, 32, 32, 32, 32, 32, 33, 33]
    assert all(a[0] + a[1] == b[0] for a, b in zip(rr, rr[1:]))
    rr = row_ranges(65536, 8, lighter=(3, 1))
    assert rr[3][1] == 31 * 256 and rr[7][1] == 33 * 256 and all(a[0] + a[1] == b[0] for a, b in zip(rr, rr[1:]))
    assert row_ranges(300, 4, lighter=(0, 1)) == row_ranges(300, 4)          # too few blocks: unchanged


def test_panel_plan():
    assert panel_plan(16384, 4) == [(0, 4096), (4096, 4096), (8192, 4096), (12288, 4096)]
    assert panel_plan(3001, 4) == [(0, 768), (768, 768), (1536, 768), (2304, 697)]
    assert panel_plan(100, 8) == [(0, 100)]
    assert [w for _, w in panel_plan(16384, "ramp")] == [1024, 3072, 4096, 4096, 4096]
    assert [w for _, w in panel_plan(16384, "ramp", align=512)] == [1024, 3072, 4096, 4096, 4096]
    assert panel_plan(3001, "ramp") == panel_plan(3001, 4)          # too narrow to ramp
    assert panel_plan(1000, [256, 512]) == [(0, 256), (256, 512), (768, 232)]
    for N in (1, 255, 257, 3001, 16384):
        for p in (1, 2, 4, 8, "ramp"):
            pl = panel_plan(N, p)
            assert sum(w for _, w in pl) == N and all(w > 0 for _, w in pl)


def test_no_cpu_compute_path():
    with pytest.raises(RuntimeError):
        ShardedGemm(8, 8, 8, torch.float32, device="cpu")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, N, K, bcast, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        def host_gemm(A, Bp, D):          # stands in for the CUDA GEMM in this CPU-only test
            D.copy_((A.double() @ Bp.double()).float())
        sg = ShardedGemm(M, N, K, torch.float32, owner=0, panels=3, device="cpu", gemm_fn=host_gemm, bcast=bcast)
        g = torch.Generator().manual_seed(1)
        A = torch.rand((M, K), generator=g) * 2 - 1
        B = torch.rand((K, N), generator=g) * 2 - 1
        sg.A.copy_(A[sg.row0:sg.row0 + sg.nrows])
        if sg.is_owner:
            sg.B.copy_(B)
        for _ in range(2):                # twice: buffers and schedule are reusable
            sg.step()
        if sg.is_owner:
            ref = (A.double() @ B.double()).float()
            out.put(bool(torch.equal(sg.D, ref)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("bcast", ["broadcast", "scatter_allgather"])
@pytest.mark.parametrize("shape", [(700, 600, 50), (256, 300, 33)])
def test_two_rank_schedule_over_gloo(shape, bcast):
    M, N, K = shape
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, M, N, K, bcast, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


# ------------------------------------------------------------------ planning of the fused (in-kernel fetch) path
def test_fetch_panel_plan_and_row_pieces():
    from decx_b200.sharded import fetch_panel_plan, row_pieces
    for N in (8, 520, 1024, 2104, 16384, 40000):
        plan = fetch_panel_plan(N)
        assert len(plan) <= 16 and plan[0][0] == 0 and sum(w for _, w in plan) == N
        assert all(c % 512 == 0 for c, _ in plan)                          # panels start on 256 x 512 tile columns
        assert all(a[0] + a[1] == b[0] for a, b in zip(plan, plan[1:]))
    for K, parts in ((16384, 7), (2053, 3), (70, 1), (16, 4), (130, 7)):
        pc = row_pieces(K, parts)
        assert len(pc) == parts and pc[0][0] == 0 and sum(n for _, n in pc) == K
        assert all(a[0] + a[1] == b[0] for a, b in zip(pc, pc[1:]))


def test_fetch_jobs_cover_b_exactly_once_and_gate_on_the_publisher():
    from decx_b200.sharded import fetch_jobs, fetch_panel_plan, row_pieces
    K, N = 2053, 2104
    panels = fetch_panel_plan(N)
    SRC, GATE, R0, NR, C0, W, P, PUB, DST, NOTIFY = range(10)
    for scatter in ("push", "pull"):
        for world, owner, active in ((2, 0, [0, 1]), (4, 0, [0, 1, 2, 3]), (8, 3, list(range(8))), (4, 0, [0, 1, 2])):
            b_ptr = [1000 * (r + 1) for r in range(world)]
            pub_ptr = [50 + 1000 * (r + 1) for r in range(world)]
            holders = [r for r in active if r != owner]
            held = {}                                                          # (rank, panel) -> rows it holds first
            owner_jobs = fetch_jobs(owner, owner, active, K, panels, b_ptr, pub_ptr, scatter)
            if scatter == "pull":
                assert owner_jobs == []
            else:
                # the owner pushes every row of every panel exactly once, each piece to one holder, flag = that holder's
                for p, (c0, w) in enumerate(panels):
                    mine = [j for j in owner_jobs if j[P] == p]
                    rows = sorted((j[R0], j[NR]) for j in mine)
                    assert rows[0][0] == 0 and sum(n for _, n in rows) == K
                    assert all(a[0] + a[1] == b[0] for a, b in zip(rows, rows[1:]))
                    assert sorted(b_ptr.index(j[DST]) for j in mine) == sorted(holders)
                    for j in mine:
                        q = b_ptr.index(j[DST])
                        assert j[SRC] == b_ptr[owner] and j[GATE] is None and j[NOTIFY] == pub_ptr[q] + 4 * p
                        assert (j[C0], j[W]) == (c0, w) and j[PUB] == 0
                        held[(q, p)] = (j[R0], j[NR])
            for r in range(world):
                jobs = fetch_jobs(r, owner, active, K, panels, b_ptr, pub_ptr, scatter)
                if r == owner:
                    continue
                if r not in active:
                    assert jobs == []
                    continue
                for p, (c0, w) in enumerate(panels):
                    mine = [j for j in jobs if j[P] == p]
                    assert all(j[C0] == c0 and j[W] == w and j[DST] is None and j[NOTIFY] is None for j in mine)
                    own = mine[0]                                              # the own piece comes first
                    if scatter == "push":
                        assert own[NR] == 0 and own[GATE] == pub_ptr[r] + 4 * p and held[(r, p)][0] == own[R0]
                        rows = sorted([held[(r, p)]] + [(j[R0], j[NR]) for j in mine[1:]])
                    else:
                        assert own[SRC] == b_ptr[owner] and own[GATE] is None
                        held[(r, p)] = (own[R0], own[NR])
                        rows = sorted((j[R0], j[NR]) for j in mine)
                    assert rows[0][0] == 0 and sum(n for _, n in rows) == K    # every row of the panel, once
                    assert all(a[0] + a[1] == b[0] for a, b in zip(rows, rows[1:]))
            # a gated pull reads exactly the rows its source holds first, behind that source's flag for the panel
            for r in range(world):
                if r == owner:
                    continue
                for j in fetch_jobs(r, owner, active, K, panels, b_ptr, pub_ptr, scatter):
                    if j[GATE] is not None and j[NR]:
                        src_rank = b_ptr.index(j[SRC])
                        assert j[GATE] == pub_ptr[src_rank] + 4 * j[P] and j[PUB] == 0
                        assert held[(src_rank, j[P])] == (j[R0], j[NR])


def test_multicast_jobs_one_store_job_per_panel_on_the_owner():
    from decx_b200.sharded import fetch_jobs, fetch_panel_plan
    K, N = 2053, 2104
    panels = fetch_panel_plan(N)
    SRC, GATE, R0, NR, C0, W, P, PUB, DST, NOTIFY = range(10)
    world, owner, active = 4, 1, [0, 1, 3]
    b_ptr = [1000 * (r + 1) for r in range(world)]
    pub_ptr = [50 + 1000 * (r + 1) for r in range(world)]
    with pytest.raises(ValueError):
        fetch_jobs(owner, owner, active, K, panels, b_ptr, pub_ptr, "multicast")
    jobs = fetch_jobs(owner, owner, active, K, panels, b_ptr, pub_ptr, "multicast", mc_ptr=9000, mc_pub_ptr=9050)
    assert len(jobs) == len(panels)
    for p, ((c0, w), j) in enumerate(zip(panels, jobs)):
        assert (j[SRC], j[GATE], j[R0], j[NR], j[C0], j[W], j[P]) == (b_ptr[owner], None, 0, K, c0, w, p)
        assert j[PUB] == 2 and j[DST] == 9000 and j[NOTIFY] == 9050 + 4 * p
    for r in (0, 3):
        jobs = fetch_jobs(r, owner, active, K, panels, b_ptr, pub_ptr, "multicast", mc_ptr=9000, mc_pub_ptr=9050)
        assert [(j[NR], j[GATE], j[P], j[DST]) for j in jobs] == [(0, pub_ptr[r] + 4 * p, p, None) for p in range(len(panels))]
    assert fetch_jobs(2, owner, active, K, panels, b_ptr, pub_ptr, "multicast", mc_ptr=9000, mc_pub_ptr=9050) == []
