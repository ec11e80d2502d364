"""Optimizers and learning-rate schedulers of the example workloads."""
from .lamb import FusedLAMB

__all__ = ["FusedLAMB"]
