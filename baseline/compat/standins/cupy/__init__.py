"""Minimal stand-in for the part of CuPy that the reference's kernel loader touches
(``communication/compressors/cupy_kernel.py:1-3,28-45``): ``cupy.cuda.function.Module`` and
``cupy.cuda.device.Device().compute_capability``.  Real CuPy is not installed in this image."""
from . import cuda  # noqa: F401

__version__ = "0.0-standin"
