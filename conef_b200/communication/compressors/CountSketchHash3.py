"""Alias module: ``DenseCSHash3`` as in ``communication/compressors/CountSketchHash3.py``."""
from ...compressors.count_sketch import DenseCSHash3  # noqa: F401
