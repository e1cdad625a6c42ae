"""GPU test of decxb200_gemm_fp32_noalloc, the fp32 GEMM for callers that cannot allocate.

It is called through the C ABI with nothing but input and output pointers and must give exactly what
the ordinary entry point (caller-provided workspace) gives for the same operands: both run the same
split pass and the same 3xTF32 kernel, so the comparison is bit for bit, and the result is checked
against the CPU oracle with this path's usual limit (metric <= 1e-5) as well.  Two calls in a row use
the library's fixed scratch array one after the other: a large problem first, then a smaller, ragged
one that lands on top of the first one's leftovers.  This file sorts last so that a run which stops at
its first failure has already executed every other test.
"""
import numpy as np
import pytest

from oracle import binding as ob
from util import make_inputs, pitch_elems

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _pitched(t, dev):
    r, c = t.shape
    buf = torch.zeros((r, pitch_elems(c, 4)), dtype=torch.float32, device=dev)
    buf[:, :c] = t.to(dev)
    return buf[:, :c]


def _noalloc(capi, A, B, C, alpha, beta, out, status):
    import ctypes
    a = (ctypes.c_float * 1)(alpha)
    b = (ctypes.c_float * 1)(beta)
    stream = torch.cuda.current_stream().cuda_stream
    return capi.lib.decxb200_gemm_fp32_noalloc(
        stream, A.shape[0], B.shape[1], A.shape[1], A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0),
        C.data_ptr() if C is not None else None, C.stride(0) if C is not None else 0,
        out.data_ptr(), out.stride(0), ctypes.cast(a, ctypes.c_void_p), ctypes.cast(b, ctypes.c_void_p),
        status.data_ptr())


def test_noalloc_matches_workspace_entry_point_on_two_calls_in_a_row():
    from decx_b200 import capi, gemm as G
    dev = torch.device("cuda:0")
    status = G.new_status(dev)
    # (M, N, K, fused): the first fills the fixed scratch array completely (1024^3 needs all 16 MiB)
    for M, N, K, fused in [(1024, 1024, 1024, False), (333, 215, 77, True)]:
        assert capi.workspace_bytes(capi.FP32, M, N, K) <= capi.NOALLOC_SCRATCH_BYTES
        A, B, C = make_inputs(np.float32, M, N, K, seed=M + K, dist="normal", with_c=fused)
        tA, tB = _pitched(torch.from_numpy(A), dev), _pitched(torch.from_numpy(B), dev)
        tC = _pitched(torch.from_numpy(C), dev) if fused else None
        alpha, beta = (0.5, -2.0) if fused else (1.0, 0.0)
        out = _pitched(torch.zeros((M, N)), dev)
        rc = _noalloc(capi, tA, tB, tC, alpha, beta, out, status)
        assert rc == 0, capi.lib.decxb200_strerror(rc).decode()
        expect = G.gemm(tA, tB, tC, alpha, beta if fused else None, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(out, expect), "no-alloc entry point differs from the workspace entry point"
        m = ob.metric(out.cpu().numpy(), ob.gemm(A, B, C, alpha, beta), A, B)
        assert m <= 1e-5, f"metric {m:.3e}"


def test_noalloc_rejects_problems_beyond_its_scratch():
    from decx_b200 import capi, gemm as G
    dev = torch.device("cuda:0")
    status = G.new_status(dev)
    M = N = K = 1056                      # needs more than the 16 MiB the library holds
    assert capi.workspace_bytes(capi.FP32, M, N, K) > capi.NOALLOC_SCRATCH_BYTES
    z = torch.zeros((M, K), device=dev)
    out = torch.full((M, N), 7.0, device=dev)
    rc = _noalloc(capi, z, z, None, 1.0, 0.0, out, status)
    torch.cuda.synchronize()
    assert rc == -5 and b"extent" in capi.lib.decxb200_strerror(rc)
    assert bool((out == 7.0).all()), "a rejected call must not touch the output"
