"""Adam with decoupled weight decay, built-in warm-up schedule and gradient-norm clipping,
without bias correction: the ``BertAdam`` of the original BERT fine-tuning recipes
(reference: ``examples/BertPretraining/optimization.py:64-174``, which cannot even be
imported without apex)."""
import math

import torch
from torch.nn.utils import clip_grad_norm_
from torch.optim import Optimizer


def warmup_cosine(x, warmup=0.002):
    return x / warmup if x < warmup else 0.5 * (1.0 + math.cos(math.pi * x))


def warmup_constant(x, warmup=0.002):
    return x / warmup if x < warmup else 1.0


def warmup_linear(x, warmup=0.002):
    return x / warmup if x < warmup else max((x - 1.0) / (warmup - 1.0), 0.0)


def warmup_poly(x, warmup=0.002, degree=0.5):
    return x / warmup if x < warmup else (1.0 - x) ** degree


SCHEDULES = {"warmup_cosine": warmup_cosine, "warmup_constant": warmup_constant, "warmup_linear": warmup_linear,
             "warmup_poly": warmup_poly}


class BertAdam(Optimizer):
    def __init__(self, params, lr, warmup=-1, t_total=-1, schedule="warmup_linear", b1=0.9, b2=0.999, e=1e-6,
                 weight_decay=0.01, max_grad_norm=1.0):
        if lr < 0 or not 0 <= b1 < 1 or not 0 <= b2 < 1 or e < 0:
            raise ValueError("invalid BertAdam hyper-parameter")
        if schedule not in SCHEDULES:
            raise ValueError(f"unknown schedule {schedule!r}")
        if not (warmup == -1 or 0.0 <= warmup < 1.0):
            raise ValueError("warmup must be -1 or in [0, 1)")
        super().__init__(params, dict(lr=lr, schedule=schedule, warmup=warmup, t_total=t_total, b1=b1, b2=b2, e=e,
                                      weight_decay=weight_decay, max_grad_norm=max_grad_norm))

    def get_lr(self):
        out = []
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state[p]
                if not st:
                    return [0]
                if group["t_total"] != -1:
                    out.append(group["lr"] * SCHEDULES[group["schedule"]](st["step"] / group["t_total"], group["warmup"]))
                else:
                    out.append(group["lr"])
        return out

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("BertAdam does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["next_m"] = torch.zeros_like(p)
                    st["next_v"] = torch.zeros_like(p)
                if group["max_grad_norm"] > 0:
                    clip_grad_norm_(p, group["max_grad_norm"])
                g = p.grad
                st["next_m"].mul_(group["b1"]).add_(g, alpha=1 - group["b1"])
                st["next_v"].mul_(group["b2"]).addcmul_(g, g, value=1 - group["b2"])
                update = st["next_m"] / (st["next_v"].sqrt() + group["e"])
                if group["weight_decay"] > 0:
                    update = update + group["weight_decay"] * p
                lr = group["lr"]
                if group["t_total"] != -1:
                    lr *= SCHEDULES[group["schedule"]](st["step"] / group["t_total"], group["warmup"])
                p.add_(update, alpha=-lr)
                st["step"] += 1
        return loss
