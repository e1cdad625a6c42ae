"""GPU tests of the panel-gated fp16 GEMM (one launch over a B that arrives in column panels)."""
import os
import subprocess
import sys
import time

import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _problem(dev, M=1024, N=2048, K=512):
    g = torch.Generator(device=dev).manual_seed(11)
    A = (torch.randn(M, K, device=dev, generator=g) * 0.1).half()
    B = (torch.randn(K, N, device=dev, generator=g) * 0.1).half()
    return A, B


@pytest.mark.parametrize("ends", [[2048], [512, 2048], [256, 768, 2048], [512, 1024, 1536, 2000]])
def test_flags_already_set_equals_plain_gemm(ends):
    from decx_b200 import gemm as G
    dev = torch.device("cuda:0")
    A, B = _problem(dev, N=ends[-1])
    st = G.new_status(dev)
    flags = torch.full((8,), 5, dtype=torch.int32, device=dev)
    out = torch.empty((A.shape[0], ends[-1]), dtype=torch.float16, device=dev)
    G.gemm_fp16_panels(A, B, out, ends, flags, 5, status=st)
    ref = G.gemm(A, B, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and torch.equal(out, ref)


def test_kernel_waits_for_panels_delivered_by_another_stream():
    """The GEMM is launched first; B's panels are copied in and flagged afterwards, out of order of need."""
    from decx_b200 import gemm as G
    dev = torch.device("cuda:0")
    A, B = _problem(dev, M=2048, N=4096, K=1024)
    ends = [512, 1536, 2560, 4096]
    Bdst = torch.zeros_like(B)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    st = G.new_status(dev)
    out = torch.empty((2048, 4096), dtype=torch.float16, device=dev)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(dev)
    G.gemm_fp16_panels(A, Bdst, out, ends, flags, 1, status=st)     # its loader waits until panel 0 arrives
    time.sleep(0.05)
    lo = 0
    with torch.cuda.stream(side):
        for i, hi in enumerate(ends):
            G.copy2d(Bdst.data_ptr() + 2 * lo, 2 * 4096, B.data_ptr() + 2 * lo, 2 * 4096, 2 * (hi - lo), 1024, side)
            G.write_flag(flags, i, 1, side)
            lo = hi
            time.sleep(0.01)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ref = G.gemm(A, B)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


def test_missing_panel_times_out_with_a_status_code():
    """A flag that nothing sets: the bounded wait expires, the kernel unwinds and reports 0x106; the context
    stays usable.  Runs in a child process so that the short wait limit does not leak into other tests."""
    code = r'''
import sys, torch
sys.path.insert(0, %r)
from decx_b200 import gemm as G
dev = torch.device("cuda:0")
A = torch.zeros(512, 256, dtype=torch.float16, device=dev); B = torch.zeros(256, 1024, dtype=torch.float16, device=dev)
out = torch.empty(512, 1024, dtype=torch.float16, device=dev)
flags = torch.zeros(8, dtype=torch.int32, device=dev); st = G.new_status(dev)
flags[0] = 7
G.gemm_fp16_panels(A, B, out, [512, 1024], flags, 7, status=st)    # panel 1 never arrives
torch.cuda.synchronize()
print("STATUS", hex(int(st.item()) & 0xffffffff))
st.zero_(); flags.fill_(8)
G.gemm_fp16_panels(A, B, out, [512, 1024], flags, 8, status=st)    # the same context still works
torch.cuda.synchronize()
print("AGAIN", int(st.item()), bool((out == 0).all()))
''' % ROOT
    env = dict(os.environ, DECXB200_WAIT_LIMIT_MS="300")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env)
    assert "STATUS 0x106" in r.stdout, r.stdout + r.stderr
    assert "AGAIN 0 True" in r.stdout, r.stdout + r.stderr
