"""decx_b200: B200-native (sm_100a) replacement for DECX's de::blas::cuda::GEMM path.

Sub-modules:
  build     in-tree nvcc / g++ build of the libraries (importable without them)
  capi      ctypes binding of the C ABI (raises ImportError if the CUDA library is missing)
  gemm      device-tensor front end used by tests and the benchmark
  sharded   row-sharded multi-GPU GEMM (one process per GPU, torch.distributed)
There is no CPU or PyTorch fallback anywhere in the package.
"""

__all__ = ["build", "capi", "gemm", "sharded"]
