"""Gradient accumulation with ONE all-reduce per optimizer step, outside DDP.

Counterpart of the reference's ``--allreduce_post_accumulation`` /
``--allreduce_post_accumulation_fp16`` mode
(``examples/BertPretraining/run_pretraining_conef.py:371-373,492-497,506-556``): the model is not
wrapped in DistributedDataParallel; every rank accumulates the gradients of its micro-batches
locally, and before the optimizer step all gradients are flattened into one buffer (fp32, or fp16
to halve the bytes on the wire), pre-divided so that the sum is the average, summed over the ranks
with a single collective and copied back.  The reference does the flatten / scale / unflatten with
apex's ``apex_C.unflatten`` and ``amp_C.multi_tensor_scale``; here they are ``torch._foreach``
calls on views of a persistent flat buffer.  This mode and the compression hooks exclude each
other (hooks need DDP's buckets), as in the reference.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch
import torch.distributed as dist


def broadcast_parameters(module: torch.nn.Module, src: int = 0, group=None) -> None:
    """What DDP's constructor does for the replicas: every rank starts from rank ``src``'s weights
    and buffers (``flat_dist_call(..., broadcast, (0,))``, run_pretraining_conef.py:497)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    tensors = [p.data for p in module.parameters()] + [b.data for b in module.buffers()]
    by_type = {}
    for t in tensors:
        by_type.setdefault((t.dtype, t.device), []).append(t)
    for ts in by_type.values():
        flat = torch.cat([t.reshape(-1) for t in ts])
        dist.broadcast(flat, src, group=group)
        off = 0
        for t in ts:
            t.copy_(flat[off : off + t.numel()].view_as(t))
            off += t.numel()


class PostAccumulationAllReduce:
    """``reducer.allreduce()`` between the last ``backward()`` of an accumulation window and
    ``optimizer.step()``.

    ``wire_dtype``: ``torch.float32`` or ``torch.float16`` / ``torch.bfloat16`` (half the bytes;
    the pre-division happens in fp32 before the cast, so the cast cannot overflow where the fp32
    gradients were finite and the average fits the half type).  ``accumulation_steps`` divides as
    well when the caller did not already scale its micro-batch losses (``predivide_accumulation``).
    Returns False (and leaves the gradients unscaled) when a non-finite value is found after the
    reduction, so that the caller can skip the step as the reference does on overflow.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], group=None, wire_dtype: torch.dtype = torch.float32,
                 accumulation_steps: int = 1, predivide_accumulation: bool = False):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        self.group = group
        self.wire_dtype = wire_dtype
        self.divisor_extra = float(accumulation_steps) if predivide_accumulation else 1.0
        self._flat: Optional[torch.Tensor] = None
        self._views: List[torch.Tensor] = []
        self._layout = None
        self.bytes_on_wire = 0

    def _buffers(self, grads: List[torch.Tensor]):
        layout = tuple((g.numel(), g.device) for g in grads)
        if layout != self._layout:
            total = sum(g.numel() for g in grads)
            self._flat = torch.empty(total, dtype=self.wire_dtype, device=grads[0].device)
            self._views, off = [], 0
            for g in grads:
                self._views.append(self._flat[off : off + g.numel()].view_as(g))
                off += g.numel()
            self._layout = layout
        return self._flat, self._views

    @torch.no_grad()
    def allreduce(self) -> bool:
        grads = [p.grad for p in self.params if p.grad is not None]
        if not grads:
            return True
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        flat, views = self._buffers(grads)
        torch._foreach_mul_(grads, 1.0 / (world * self.divisor_extra))     # pre-division in fp32
        torch._foreach_copy_(views, grads)                                  # flatten (+ cast to the wire type)
        if world > 1:
            dist.all_reduce(flat, group=self.group)
        self.bytes_on_wire = flat.numel() * flat.element_size()
        finite = bool(torch.isfinite(flat).all()) if self.wire_dtype != torch.float32 else True
        torch._foreach_copy_(grads, views)                                  # unflatten (+ cast back)
        return finite
