"""The C++ drop-in (namespace de) is tested by C++ programs under tests/cpp, built by decx_b200.build:
host_units (CPU: ABI sizes, pitch rules, host matrix, half conversion, errors, the device pool on a fake
allocator) and gemm_api (GPU: a DECX-style user program through de::blas::cuda::GEMM)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")


def _run(name, timeout=600):
    r = subprocess.run([os.path.join(CPP, name + ".bin")], capture_output=True, text=True, timeout=timeout)
    print(r.stdout[-4000:], r.stderr[-2000:])
    return r


def test_host_units_cpu():
    r = _run("host_units")
    assert r.returncode == 0 and "all checks passed" in r.stdout


def test_drop_in_exports_the_reference_symbols():
    """Mangled names a program compiled against DECX's headers would import for this path."""
    out = subprocess.run(["nm", "-D", "--defined-only", os.path.join(ROOT, "decx_b200", "host", "libDECX_b200.so")],
                         capture_output=True, text=True, check=True).stdout
    for sym in [
        "_ZN2de4blas4cuda4GEMMERNS_10GPU_MatrixES3_S3_",
        "_ZN2de4blas4cuda4GEMMERNS_10GPU_MatrixES3_S3_S3_NS_6NumberES4_",
        "_ZN2de4blas4cuda4GEMMERNS_6MatrixES3_S3_",
        "_ZN2de4blas4cuda4GEMMERNS_6MatrixES3_S3_S3_",
        "_ZN2de18CreateGPUMatrixRefENS_18_DATA_TYPES_FLAGS_EjjNS_14_DATA_FORMATS_E",
        "_ZN2de15CreateMatrixRefENS_18_DATA_TYPES_FLAGS_EjjNS_14_DATA_FORMATS_E",
        "_ZN2de6MemcpyERNS_6MatrixERNS_10GPU_MatrixENS_7Point2DES4_S4_i",
        "_ZN2de8InitCudaEv", "_ZN2de11InitCPUInfoEv", "_ZN2de4cuda14DECX_CUDA_exitEv",
        "_ZN2de3cpu19DecxSetThreadingNumEm", "_ZN2de12GetLastErrorEv",
        "_ZN2de10Float2HalfERKf", "_ZN2de10Half2FloatERKNS_4HalfE",
        "_ZN2de4cuda9PinMemoryERNS_6MatrixE", "_ZN2de4cuda11UnpinMemoryERNS_6MatrixE",
    ]:
        assert sym in out, f"{sym} is not exported"


REF_INC = "/root/reference/srcs/includes"


@pytest.mark.skipif(not os.path.isdir(REF_INC), reason="reference headers not mounted")
def test_program_built_against_reference_headers_runs_on_the_drop_in(tmp_path):
    """ABI check: a program compiled with the reference's public headers links and runs against libDECX_b200."""
    host, csrc = os.path.join(ROOT, "decx_b200", "host"), os.path.join(ROOT, "decx_b200", "csrc")
    exe = str(tmp_path / "abi_probe")
    subprocess.run(["g++", "-std=c++17", "-include", "cstdint", "-I", REF_INC,
                    os.path.join(ROOT, "tests", "cpp_abi", "abi_probe.cxx"), "-o", exe, "-L", host, "-lDECX_b200",
                    "-L", csrc, "-ldecx_b200", f"-Wl,-rpath,{host}", f"-Wl,-rpath,{csrc}"], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and "abi probe ok" in r.stdout


@pytest.mark.gpu
def test_gemm_api_gpu():
    r = _run("gemm_api")
    assert r.returncode == 0 and "all checks passed" in r.stdout
