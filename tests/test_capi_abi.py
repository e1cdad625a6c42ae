"""CPU tests of the C-ABI library: it loads without a GPU, exports every symbol the header
declares, and rejects bad arguments before touching CUDA."""
import ctypes
import os
import re

from decx_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            names |= set(re.findall(r"DECXB200_API[^;(]*?\b(decxb200_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    declared = _declared()
    assert declared, "no declarations found in include/*.h"
    for name in sorted(declared):
        assert hasattr(capi.lib, name), f"{name} is declared in include/ but not exported"
    assert declared == set(capi.EXPORTS), "decx_b200/capi.py and include/decx_b200.h disagree"


def test_version_and_strerror():
    assert capi.lib.decxb200_version().decode().count(".") == 1
    assert capi.lib.decxb200_strerror(0) == b"success"
    for code in (-1, -2, -3, -4, -5, -6):
        assert len(capi.lib.decxb200_strerror(code)) > 10


def test_workspace_sizes():
    ws = capi.workspace_bytes
    assert ws(capi.FP16, 4096, 4096, 4096) == 0
    # fp32: (hi, lo) planes of A (M x K) and B (K x N), rows padded to 32 floats
    assert ws(capi.FP32, 8192, 8192, 8192) == 4 * 8192 * 8192 * 4
    assert ws(capi.FP32, 5, 3, 7) == 2 * 768 + 2 * 1024   # 640- and 896-byte planes padded to 256 B
    # cplxf: A viewed as M x 2K floats, B expanded to 2K x 2N floats
    assert ws(capi.CPLXF, 4096, 4096, 4096) == 2 * 4096 * 8192 * 4 + 2 * 8192 * 8192 * 4
    assert ws(capi.FP32, 0, 4, 4) == 0
    assert capi.lib.decxb200_gemm_host_arena_bytes(capi.FP16, 0, 1, 1, 0) == 0
    assert capi.lib.decxb200_gemm_host_arena_bytes(capi.FP16, 4096, 4096, 4096, 0) > 3 * 4096 * 4096 * 2 // 2


def test_bad_arguments_are_rejected_without_a_gpu():
    g = capi.lib.decxb200_gemm
    buf = (ctypes.c_float * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    args = lambda dt, M, N, K, A, B, D, lda=8, ldb=8, ldd=8: (dt, None, M, N, K, A, lda, B, ldb, None, 0, D, ldd,
                                                              None, None, None, 0, None)
    assert g(*args(4, 4, 4, 4, p, p, p)) == -1            # unknown dtype (4 = int32: no GEMM)
    assert g(*args(capi.FP32, 0, 4, 4, p, p, p)) == -1    # zero extent
    assert g(*args(capi.FP32, 4, 4, 4, None, p, p)) == -1  # null operand
    assert g(*args(capi.FP32, 4, 4, 4, p, p, p, lda=3)) == -1  # pitch smaller than width
    assert capi.lib.decxb200_gemm_ex(*args(capi.FP32, 4, 4, 4, p, p, p), 3, 0) == -1  # bad cta_group


def test_header_is_plain_c(tmp_path):
    """include/decx_b200.h is a C header: it must compile as C99 on its own."""
    import subprocess
    src = tmp_path / "use.c"
    src.write_text('#include "decx_b200.h"\nint main(void) { return decxb200_gemm_workspace_bytes(DECXB200_FP16, 1, 1, 1) != 0; }\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), "-c", str(src),
                    "-o", str(tmp_path / "use.o")], check=True)


def test_front_end_refuses_host_tensors_and_missing_gpu():
    """No fallback: the device front end rejects CPU tensors instead of computing on the host."""
    import pytest
    import torch
    from decx_b200 import gemm as G
    with pytest.raises(RuntimeError):
        G.gemm(torch.zeros(4, 4), torch.zeros(4, 4))
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            G.gemm_host(torch.zeros(4, 4), torch.zeros(4, 4))


def test_multi_gpu_host_plan_partitions_rows_pieces_and_panels():
    """The planner of the in-process multi-GPU host GEMM, on the CPU: rows of A in whole 256-row tiles, B's rows
    dealt once over the devices that have work, panels that tile the columns on 512-column boundaries."""
    u32 = ctypes.c_uint32
    for n, M, N, K in ((1, 300, 520, 70), (2, 1300, 2104, 520), (8, 65536, 16384, 16384), (4, 520, 1024, 256),
                       (8, 700, 40000, 2053), (3, 100000, 8, 16)):
        row0, nrows, rb, p0, pr = ((u32 * n)() for _ in range(5))
        npan, pend = u32(), (u32 * 16)()
        assert capi.lib.decxb200_gemm_host_multi_plan(n, M, N, K, row0, nrows, rb, p0, pr, ctypes.byref(npan), pend) == 0
        assert sum(nrows) == M and row0[0] == 0
        covered = 0
        for d in range(n):
            if nrows[d]:
                assert row0[d] == covered and row0[d] % 256 == 0 and 0 < rb[d] <= nrows[d]
                assert rb[d] == nrows[d] or rb[d] % 256 == 0
                covered += nrows[d]
        pieces = sorted((p0[d], pr[d]) for d in range(n) if nrows[d])
        assert pieces[0][0] == 0 and sum(r for _, r in pieces) == K          # every row of B uploaded exactly once
        assert all(a[0] + a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
        assert all(pr[d] == 0 for d in range(n) if not nrows[d])             # idle devices upload nothing
        ends = list(pend[: npan.value])
        assert 1 <= npan.value <= 16 and ends[-1] == N and ends == sorted(set(ends))
        assert all(e % 512 == 0 for e in ends[:-1])
        assert capi.lib.decxb200_gemm_host_multi_arena_bytes(capi.FP16, n, M, N, K) > K * N * 2
    assert capi.lib.decxb200_gemm_host_multi_plan(0, 1, 1, 1, None, None, None, None, None, None, None) == -1
