"""Alias module: fp16-storage ``DenseCS`` as in ``communication/compressors/halfCountSketch.py``."""
from ...compressors.count_sketch import HalfDenseCS as DenseCS  # noqa: F401
