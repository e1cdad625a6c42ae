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
        # Vector overloads of GEMM, Transpose, TypeCast, vectors and their Memcpy
        "_ZN2de4blas4cuda4GEMMERNS_6VectorERNS_6MatrixES3_j", "_ZN2de4blas4cuda4GEMMERNS_6MatrixERNS_6VectorES5_j",
        "_ZN2de4cuda9TransposeERNS_10GPU_MatrixES2_", "_ZN2de4cuda8TypeCastERNS_10GPU_MatrixES2_i",
        "_ZN2de15CreateVectorRefENS_18_DATA_TYPES_FLAGS_Em", "_ZN2de18CreateGPUVectorRefENS_18_DATA_TYPES_FLAGS_Em",
        "_ZN2de6MemcpyERNS_6VectorERNS_10GPU_VectorEmmmi",
        # services other DECX modules link against
        "_ZN4decx5alloc8_alloc_DEPPNS_8MemBlockEm", "_ZN4decx5alloc10_dealloc_DEPNS_8MemBlockE",
        "_ZN4decx5alloc19_alloc_D_same_placeEPPNS_8MemBlockE", "_ZN4decx5alloc8Memset_DEPNS_8MemBlockEmiPP11CUstream_st",
        "_ZN4decx4cuda19get_cuda_stream_refEi", "_ZN4decx4cuda18get_cuda_event_refEi",
        "_ZN4decx15ResourceCheckInEPPvlPFvS0_E", "_ZN4decx12ResourceLockEm", "_ZN4decx14ResourceUnlockEm",
        "_ZN4decx16ResourceCheckOutEm",
    ]:
        assert sym in out, f"{sym} is not exported"


@pytest.mark.parametrize("san", ["address,undefined", "thread"])
def test_host_units_under_sanitizers(tmp_path, san):
    """The host layer's sources compiled WITH the sanitizer (not the shipped .so) and the same unit tests run on
    them: heap misuse / undefined behaviour in the pool, containers and resource manager, and data races between
    the collector thread and its users."""
    host = os.path.join(ROOT, "decx_b200", "host")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    srcs = [os.path.join(host, f) for f in sorted(os.listdir(host)) if f.endswith(".cpp") and f not in ("gemm_api.cpp", "blas_aux.cpp", "multi_gpu.cpp", "conv_api.cpp")]
    stub = tmp_path / "abi_stub.cpp"       # the unit tests call the GEMM entry only to see its "not initialised" error
    stub.write_text('#include "DECX.h"\n#include "decx_b200/host/internal.h"\n'
                    'void de::blas::cuda::GEMM(de::Matrix&, de::Matrix&, de::Matrix&) {\n'
                    '    decx::err::set(de::GetLastError(), de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first"); }\n'
                    'de::DH de::nn::cuda::Conv2D(de::GPU_Tensor&, de::GPU_TensorArray&, de::GPU_Tensor&, const de::Point2D, const de::extend_label) {\n'
                    '    de::DH h; decx::err::set(&h, de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first"); return h; }\n'
                    'void de::blas::cuda::GEMM(de::Matrix&, de::Matrix&, de::Matrix&, de::Matrix&) {\n'
                    '    decx::err::set(de::GetLastError(), de::DECX_FAIL_CUDA_not_init, "error: CUDA should be initialized first"); }\n')
    exe = str(tmp_path / "host_units_san")
    cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={san}", "-fno-omit-frame-pointer", "-I", os.path.join(ROOT, "include"),
           "-I", ROOT, "-I", os.path.join(cuda, "include"), os.path.join(CPP, "host_units.cpp"), str(stub), *srcs, "-o", exe,
           "-L", os.path.join(cuda, "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    b = subprocess.run(cmd, capture_output=True, text=True)
    if b.returncode != 0 and ("cannot find -l" in b.stderr or "sanitizer" in b.stderr.lower() and "not supported" in b.stderr.lower()):
        pytest.skip("sanitizer runtime not installed: " + b.stderr[-200:])
    assert b.returncode == 0, b.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=0:protect_shadow_gap=0", TSAN_OPTIONS="halt_on_error=1")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    print(r.stdout[-3000:], r.stderr[-3000:])
    assert r.returncode == 0 and "all checks passed" in r.stdout
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error:" not in r.stderr and "WARNING: ThreadSanitizer" not in r.stderr


REF_INC = os.path.join(os.environ.get("DECX_REF_ROOT") or os.path.join(os.path.dirname(ROOT), "reference"), "srcs", "includes")


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
