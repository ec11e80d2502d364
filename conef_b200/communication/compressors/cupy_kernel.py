"""Alias module: runtime kernel loader with the call shape of ``communication/compressors/cupy_kernel.py``."""
from ...ops.jit import JitKernel as cupyKernel  # noqa: F401
