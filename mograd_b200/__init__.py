"""mograd_b200: B200-native kernels for mograd's training hot path.

The package is a thin host layer over libmograd_b200.so (hand-written sm_100a
CUDA behind a C ABI).  Import `mograd_b200.dispatch` for the operator-level
calls; the shared object must have been built (`python -m mograd_b200.build`).
"""
from ._lib import BF16, F32, KernelError, LIB_PATH, load  # noqa: F401

__all__ = ["BF16", "F32", "KernelError", "LIB_PATH", "load"]
