"""Optimizers and learning-rate schedulers of the example workloads."""
from .bert_adam import BertAdam
from .lamb import FusedLAMB
from .sgd import FusedSGD
from .schedulers import (ConstantWarmUpScheduler, CosineWarmUpScheduler, LinearWarmUpScheduler,
                         PolyWarmUpScheduler)

__all__ = ["FusedLAMB", "FusedSGD", "BertAdam", "LinearWarmUpScheduler", "CosineWarmUpScheduler", "ConstantWarmUpScheduler",
           "PolyWarmUpScheduler"]
