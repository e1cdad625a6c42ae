"""GPU tests of the host-matrix GEMM sharded over the GPUs of one process (`decxb200_gemm_host_multi`).

With one visible GPU the call still takes the same route (row blocks, upload flags, wait-only jobs of the fetching
kernel); with several, every GPU uploads its rows of B and the others fetch them over NVLink."""
import numpy as np
import pytest

from oracle import binding as ob
from util import make_inputs

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _device_sets():
    n = torch.cuda.device_count()
    sets = [[0]]
    if n >= 2:
        sets += [[0, 1], [1, 0]]
    if n >= 4:
        sets.append([0, 1, 2, 3])
    if n >= 8:
        sets.append(list(range(8)))
    return sets


@pytest.mark.parametrize("shape", [(300, 520, 70), (1300, 2104, 520), (5000, 1024, 2304), (2048, 4096, 2048)])
def test_host_multi_matches_oracle_and_single_gpu(shape):
    from decx_b200 import gemm as G
    M, N, K = shape
    A, B, _ = make_inputs(np.float16, M, N, K, seed=M + N, dist="small")
    pad = lambda x: torch.from_numpy(np.pad(x, ((0, 0), (0, 8)))).pin_memory()[:, : x.shape[1]]     # host pitch > width
    hA, hB = pad(A), pad(B)
    ref = None
    for devs in _device_sets():
        out = torch.full((M, N + 8), float("nan"), dtype=torch.float16).pin_memory()
        G.gemm_host_multi(hA, hB, out=out[:, :N], devices=devs)
        assert torch.isnan(out[:, N:]).all()
        got = out[:, :N].clone()
        if ref is None:
            ref = got
            rows = sorted({0, 255, 256, M // 2, M - 1})
            assert ob.metric(got[rows].numpy(), ob.gemm(A[rows], B), A[rows], B) <= 1e-2
            single = G.gemm_host(hA, hB, device=torch.device("cuda:0"))
            assert torch.equal(single, got)                  # same kernels, same K order: same bits
        else:
            assert torch.equal(got, ref), f"devices {devs} disagree with one GPU"


def test_host_multi_argument_errors():
    from decx_b200 import capi, gemm as G
    A = torch.zeros(512, 64, dtype=torch.float16)
    with pytest.raises(capi.DecxB200Error) as e:
        G.gemm_host_multi(A, torch.zeros(64, 12, dtype=torch.float16), devices=[0])        # N not a multiple of 8
    assert e.value.code == -2
    with pytest.raises(capi.DecxB200Error) as e:
        G.gemm_host_multi(A, torch.zeros(64, 16, dtype=torch.float16), devices=[0, 0])     # the same device twice
    assert e.value.code == -1
    assert capi.lib.decxb200_gemm_host_multi_arena_bytes(capi.FP32, 2, 512, 512, 512) == 0  # fp16 only
