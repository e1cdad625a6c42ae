"""Generates tests/golden/ref_cpu_gemm.npz from the REFERENCE's own de::blas::cpu::GEMM.

Run where the reference sources are mounted (python tests/golden/make_golden.py): it builds
oracle/_ref/libdecx_ref_cpu.so from those sources (oracle/Makefile), runs one process per shape
on seeded inputs and stores inputs and outputs.  The shapes are ones on which the reference's
CPU path is known to be right: plain (unfused) fp32, and complex shapes without odd extents.
The stored outputs pin oracle/gemm_oracle.c and are compared with the CUDA path in the GPU tests.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import binding as ob  # noqa: E402

CASES = [
    # name, dtype, M, N, K, threads, seed
    ("f32_64", np.float32, 64, 64, 64, 1, 11),
    ("f32_ragged", np.float32, 257, 131, 77, 4, 12),
    ("f32_192", np.float32, 192, 160, 128, 8, 13),
    ("c64_64", np.complex64, 64, 64, 64, 1, 21),
    ("c64_128x64x46", np.complex64, 128, 64, 46, 2, 22),
    ("c64_128", np.complex64, 128, 128, 128, 8, 23),
]


def inputs(dtype, M, N, K, seed):
    rng = np.random.default_rng(seed)
    if dtype == np.complex64:
        A = (rng.uniform(-1, 1, (M, K)) + 1j * rng.uniform(-1, 1, (M, K))).astype(dtype)
        B = (rng.uniform(-1, 1, (K, N)) + 1j * rng.uniform(-1, 1, (K, N))).astype(dtype)
    else:
        A = rng.uniform(-1, 1, (M, K)).astype(dtype)
        B = rng.uniform(-1, 1, (K, N)).astype(dtype)
    return A, B


def main():
    ob.build()
    assert ob.ref_available(), "reference sources not mounted: cannot regenerate the golden file"
    out = {}
    for name, dt, M, N, K, thr, seed in CASES:
        A, B = inputs(dt, M, N, K, seed)
        D, _, used = ob.ref_cpu_gemm(A, B, threads=thr)
        m = ob.metric(D, ob.gemm(A, B), A, B)
        print(f"{name}: threads {used}, reference vs oracle metric {m:.3e}")
        assert m < 1e-5, "the reference itself is off on this shape; pick another"
        out[name + "_A"], out[name + "_B"], out[name + "_D"] = A, B, D
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cpu_gemm.npz"), **out)


if __name__ == "__main__":
    main()
