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
            "-shared", "-o", out] + [f for f in srcs if f.endswith(".cu")]
        subprocess.run(cmd, check=True, cwd=CSRC)
    return out


HOST = os.path.join(HERE, "host")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build_host(force=False):
    """The C++ drop-in (namespace de / decx) on top of the C ABI: decx_b200/host/libDECX_b200.so."""
    out = os.path.join(HOST, "libDECX_b200.so")
    srcs = [os.path.join(HOST, f) for f in sorted(os.listdir(HOST)) if f.endswith(".cpp")]
    deps = srcs + [os.path.join(HOST, "internal.h"), os.path.join(CSRC, "libdecx_b200.so")]
    for root, _, files in os.walk(os.path.join(ROOT, "include")):
        deps += [os.path.join(root, f) for f in files]
    if force or _stale(out, deps):
        cmd = [shutil.which("g++") or "g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden",
               "-I", os.path.join(CUDA_HOME, "include"), *srcs, "-o", out,
               "-L", CSRC, "-ldecx_b200", "-Wl,-rpath,$ORIGIN/../csrc",
               "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
        subprocess.run(cmd, check=True, cwd=HOST)
    return out


def build_cpp_tests(force=False):
    """The C++ programs under tests/cpp (written against include/DECX.h like a DECX user program)."""
    tdir = os.path.join(ROOT, "tests", "cpp")
    outs = []
    if not os.path.isdir(tdir):
        return outs
    lib = os.path.join(HOST, "libDECX_b200.so")
    for f in sorted(os.listdir(tdir)):
        if not f.endswith(".cpp"):
            continue
        src, out = os.path.join(tdir, f), os.path.join(tdir, f[:-4] + ".bin")
        if force or _stale(out, [src, lib]):
            cmd = [shutil.which("g++") or "g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"),
                   "-I", ROOT, "-I", os.path.join(CUDA_HOME, "include"), src, "-o", out,
                   "-L", HOST, "-lDECX_b200", "-L", CSRC, "-ldecx_b200",
                   f"-Wl,-rpath,{HOST}", f"-Wl,-rpath,{CSRC}", "-Wl,-rpath,$ORIGIN/../../decx_b200/host",
                   "-Wl,-rpath,$ORIGIN/../../decx_b200/csrc", "-lpthread"]
            subprocess.run(cmd, check=True, cwd=tdir)
        outs.append(out)
    return outs


def build_all(force=False, verbose=False):
    return [build_kernels(force, verbose), build_host(force)] + build_cpp_tests(force)


if __name__ == "__main__":
    for p in build_all(force="--force" in sys.argv, verbose="-v" in sys.argv):
        print("built", p)
