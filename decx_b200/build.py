"""In-tree build of the CUDA library (``python -m decx_b200.build``).

nvcc cross-compiles for sm_100a without a GPU.  The product is
``decx_b200/csrc/libdecx_b200.so`` (the C ABI of ``include/decx_b200.h``).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_kernels(force=False, verbose=False):
    out = os.path.join(CSRC, "libdecx_b200.so")
    srcs = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh"))]
    srcs.append(os.path.join(ROOT, "include", "decx_b200.h"))
    if force or _stale(out, srcs):
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [
            "-shared", "-o", out, os.path.join(CSRC, "capi.cu")]
        subprocess.run(cmd, check=True, cwd=CSRC)
    return out


def build_all(force=False, verbose=False):
    return [build_kernels(force, verbose)]


if __name__ == "__main__":
    for p in build_all(force="--force" in sys.argv, verbose="-v" in sys.argv):
        print("built", p)
