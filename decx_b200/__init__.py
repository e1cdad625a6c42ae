"""decx_b200: B200-native (sm_100a) replacement for DECX's de::blas::cuda::GEMM path."""
from . import capi  # noqa: F401  (raises if the CUDA library has not been built)

__all__ = ["capi"]
