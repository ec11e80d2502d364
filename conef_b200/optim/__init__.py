"""Optimizers and learning-rate schedulers of the example workloads."""
from .bert_adam import BertAdam
from .lamb import FusedLAMB
from .schedulers import (ConstantWarmUpScheduler, CosineWarmUpScheduler, LinearWarmUpScheduler,
                         PolyWarmUpScheduler)

__all__ = ["FusedLAMB", "BertAdam", "LinearWarmUpScheduler", "CosineWarmUpScheduler", "ConstantWarmUpScheduler",
           "PolyWarmUpScheduler"]
