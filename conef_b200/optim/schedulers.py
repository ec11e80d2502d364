"""Warm-up learning-rate schedules driven by the optimizer's own step counter.

Same family as the reference's ``examples/BertPretraining/schedulers.py:51-131``: the
learning rate rises linearly during the first ``warmup`` fraction of ``total_steps`` and then
follows a constant, linear, cosine or polynomial decay.  ``step()`` reads the largest
``state[p]["step"]`` of the optimizer (LAMB / Adam keep one), so that skipped optimizer
steps (overflow, accumulation) do not advance the schedule.
"""
import math

from torch.optim.lr_scheduler import _LRScheduler


class _WarmupBase(_LRScheduler):
    def __init__(self, optimizer, warmup, total_steps, last_epoch=-1):
        self.warmup = warmup
        self.total_steps = total_steps
        super().__init__(optimizer, last_epoch)

    def _progress(self) -> float:
        steps = [st.get("step", 0) for st in self.optimizer.state.values() if isinstance(st, dict)]
        step = max([int(s) for s in steps], default=0) + 1
        self.last_epoch = step
        return step / max(1, self.total_steps)

    def _factor(self, progress: float) -> float:
        raise NotImplementedError

    def get_lr(self):
        progress = self._progress()
        if self.warmup > 0 and progress < self.warmup:
            return [base * progress / self.warmup for base in self.base_lrs]
        return [base * self._factor(progress) for base in self.base_lrs]

    def step(self, epoch=None):
        for group, lr in zip(self.optimizer.param_groups, self.get_lr()):
            group["lr"] = lr
        self._last_lr = [g["lr"] for g in self.optimizer.param_groups]


class ConstantWarmUpScheduler(_WarmupBase):
    def _factor(self, progress):
        return 1.0


class LinearWarmUpScheduler(_WarmupBase):
    def _factor(self, progress):
        return max((progress - 1.0) / (self.warmup - 1.0), 0.0)


class CosineWarmUpScheduler(_WarmupBase):
    def _factor(self, progress):
        return 0.5 * (1.0 + math.cos(math.pi * min(progress, 1.0)))


class PolyWarmUpScheduler(_WarmupBase):
    def __init__(self, optimizer, warmup, total_steps, degree=0.5, last_epoch=-1):
        self.degree = degree
        super().__init__(optimizer, warmup, total_steps, last_epoch)

    def _factor(self, progress):
        return (1.0 - min(progress, 1.0)) ** self.degree
