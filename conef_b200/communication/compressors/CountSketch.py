"""Alias module: ``DenseCS`` as in the reference's ``communication/compressors/CountSketch.py``."""
from ...compressors.count_sketch import DenseCS  # noqa: F401
