"""Multi-GPU test of the row-sharded GEMM (needs >= 2 GPUs; skipped on a single-GPU box).

Ranks run as child processes over NCCL.  The sharded result must equal the single-GPU result of
the same kernel bit for bit (same tiles, same K order), in both gather modes."""
import os
import socket
import sys

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, N, K, dtype_name, gather, bcast, out, overlap=None, tile=0, expect_overlap=None,
            scatter="push"):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from decx_b200 import gemm as G
        from decx_b200.sharded import ShardedGemm
        dtype = getattr(torch, dtype_name)
        g = torch.Generator(device=dev).manual_seed(3)
        if dtype == torch.complex64:
            mk = lambda r, c: torch.complex(torch.rand((r, c), device=dev, generator=g) * 2 - 1,
                                            torch.rand((r, c), device=dev, generator=g) * 2 - 1)
        else:
            mk = lambda r, c: (torch.rand((r, c), device=dev, generator=g) * 2 - 1).to(dtype)
        A, B = mk(M, K), mk(K, N)                     # same seed on every rank: identical full inputs
        sg = ShardedGemm(M, N, K, dtype, owner=0, panels=3 if overlap != "fused" else "ramp", gather=gather, device=dev,
                         bcast=bcast, overlap=overlap, tile=tile, scatter=scatter)
        if expect_overlap is not None:
            assert sg.overlap == expect_overlap, (sg.overlap, expect_overlap)
        sg.A.copy_(A[sg.row0:sg.row0 + sg.nrows])
        if sg.is_owner:
            sg.B.copy_(B)
        for _ in range(3):
            if sg.is_owner:
                sg.D.zero_()
            sg.step()
        torch.cuda.synchronize(dev)
        ok = int(sg.status.item()) == 0
        if tile == 3 and sg.nrows:
            ok = ok and sg.kernel_variant % 100 == 22          # the 256 x 512 tile really ran
        if sg.overlap == "fused" and not sg.is_owner and sg.nrows:
            ok = ok and bool(torch.equal(sg.Bfull, B))         # the couriers completed this rank's replica
        if sg.is_owner:
            single = G.gemm(A, B)
            torch.cuda.synchronize(dev)
            ok = ok and bool(torch.equal(sg.D, single))
            from oracle import binding as ob                   # and the oracle agrees on sampled rows
            rows = sorted({0, 255, 256, M // 2, M - 1})
            ref = ob.gemm(A[rows].cpu().numpy(), B.cpu().numpy())
            m = ob.metric(sg.D[rows].cpu().numpy(), ref, A[rows].cpu().numpy(), B.cpu().numpy())
            ok = ok and m <= {"float16": 1e-2}.get(dtype_name, 1e-5)
            out.put(ok)
        sg.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("gather", ["peer", "collective"])
@pytest.mark.parametrize("dtype_name,shape", [("float16", (2048, 1536, 512)), ("float16", (1300, 2104, 256)), ("float32", (1100, 700, 304)),
                                              ("complex64", (600, 520, 130))])
def test_sharded_equals_single_gpu(dtype_name, shape, gather):
    # every way of moving B gets covered: p2p needs K to be a multiple of the rank count, else NCCL is used
    bcast = {"peer": "p2p", "collective": "scatter_allgather" if dtype_name == "float32" else "broadcast"}[gather]
    world = min(torch.cuda.device_count(), 4)
    M, N, K = shape
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, dtype_name, gather, bcast, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


FUSED_CASES = [
    # shape, overlap, tile, what must have been selected
    ((2048, 1536, 512), None, 0, "fused"),
    ((1300, 2104, 2304), None, 3, "fused"),          # ragged M and N on the 256 x 512 tile, K >= 2048
    ((2048, 4096, 2048), "fused", 3, "fused"),
    ((2048, 4096, 2048), "single", 3, "single"),     # copy-engine delivery + flag-gated wide tile
    ((520, 1024, 256), None, 0, "fused"),            # fewer row blocks than ranks can occur at 4 GPUs
    ((1300, 2104, 2304), None, 3, "fused", "pull"),       # receivers load their pieces from the owner
    ((1300, 2104, 2304), None, 3, "fused", "multicast"),  # the owner stores through the NVLink multicast mapping
    ((2048, 4096, 2048), "fused", 0, "fused", "multicast"),
]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("case", FUSED_CASES)
def test_fp16_single_launch_paths_equal_single_gpu(case):
    """fp16 with the broadcast of B inside the step's one launch: the kernel-fetched ("fused") and the
    copy-engine-fed ("single") forms, also on the 256 x 512 tile the large configurations run."""
    shape, overlap, tile, expect = case[:4]
    scatter = case[4] if len(case) > 4 else "push"
    world = min(torch.cuda.device_count(), 4)
    M, N, K = shape
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, "float16", "peer", "p2p", q, overlap, tile, expect,
                                               scatter))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True
