"""Numerical ops: ``reference`` (PyTorch oracle / CPU path) and ``native`` (sm_100a kernels)."""
from . import native, reference

__all__ = ["native", "reference"]
