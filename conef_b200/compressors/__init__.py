"""Error compressors: what the error-feedback buffer is stored as."""
from .count_sketch import DenseCS, DenseCSHash3, HalfDenseCS, tables_for
from .other import (ERROR_COMPRESSORS, DenseError, LowRankError, Quant8Error, TopKError,
                    make_error_compressor)

__all__ = ["DenseCS", "DenseCSHash3", "HalfDenseCS", "DenseError", "TopKError", "Quant8Error",
           "LowRankError", "ERROR_COMPRESSORS", "make_error_compressor", "tables_for"]
