"""A small data-parallel training front end: model + optimizer + reducer in one object.

This is the call a user makes for a whole training step::

    trainer = DataParallelTrainer(model, optimizer, loss_fn, reducer=args_or_state_hook,
                                  autocast_dtype=torch.bfloat16)
    loss = trainer.step(inputs, target)          # host (pinned) or device tensors

It wraps the model in ``DistributedDataParallel`` (one process per GPU),
registers the communication hook selected by the reducer, moves host inputs
to the device with non-blocking copies, runs forward / backward (the hook
compresses each gradient bucket on a side stream while backward continues)
and the optimizer step.  It plays the role of the reference's per-example
training loops (examples/ImageClassification/main.py:211-235,260-314).
"""
from __future__ import annotations

import contextlib
from typing import Any, Callable, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel

from .parallel.registry import build_state_and_hook


class DataParallelTrainer:
    def __init__(self, model: torch.nn.Module, optimizer_factory: Callable, loss_fn: Callable, *,
                 reducer: Union[None, Any, Tuple[Any, Callable]] = None, device: Optional[torch.device] = None,
                 autocast_dtype: Optional[torch.dtype] = None, bucket_cap_mb: float = 25.0,
                 channels_last: bool = False, grad_clip: Optional[float] = None,
                 forward_fn: Optional[Callable] = None):
        """``reducer`` is ``None`` (plain all-reduce), an argparse-like namespace with
        ``grad_reducer`` etc. (see :func:`conef_b200.get_comm_hooks`), or a ``(state, hook)`` pair.
        ``optimizer_factory(params)`` builds the optimizer on the wrapped model's parameters.
        ``forward_fn(model, *inputs)`` customises the forward call (default ``model(*inputs)``)."""
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
                else torch.device("cpu")
        self.device = device
        model = model.to(device)
        if channels_last:
            model = model.to(memory_format=torch.channels_last)
        self.channels_last = channels_last
        ddp_kwargs = dict(bucket_cap_mb=bucket_cap_mb, gradient_as_bucket_view=True)
        if device.type == "cuda":
            ddp_kwargs.update(device_ids=[device.index], output_device=device.index)
        self.model = DistributedDataParallel(model, **ddp_kwargs)
        if reducer is None:
            self.state, hook = None, None
        elif isinstance(reducer, tuple):
            self.state, hook = reducer
            self.model.register_comm_hook(self.state, hook)
        else:
            self.state, hook = build_state_and_hook(reducer)
            if self.state is not None:
                self.model.register_comm_hook(self.state, hook)
        self.optimizer = optimizer_factory(self.model.parameters())
        self.loss_fn = loss_fn
        self.autocast_dtype = autocast_dtype
        self.grad_clip = grad_clip
        self.forward_fn = forward_fn
        self.steps = 0

    def _to_device(self, t):
        if torch.is_tensor(t):
            if t.device != self.device:
                t = t.to(self.device, non_blocking=True)
            if self.channels_last and t.dim() == 4:
                t = t.contiguous(memory_format=torch.channels_last)
        return t

    def step(self, inputs: Union[torch.Tensor, Sequence[Any]], target: Any) -> torch.Tensor:
        """One optimisation step; returns the detached loss (a device tensor)."""
        if torch.is_tensor(inputs):
            inputs = (inputs,)
        inputs = tuple(self._to_device(t) for t in inputs)
        if isinstance(target, (tuple, list)):
            target = tuple(self._to_device(t) for t in target)
        else:
            target = self._to_device(target)
        ctx = (torch.autocast(self.device.type, dtype=self.autocast_dtype)
               if self.autocast_dtype is not None else contextlib.nullcontext())
        self.optimizer.zero_grad(set_to_none=False)
        with ctx:
            out = self.forward_fn(self.model, *inputs) if self.forward_fn else self.model(*inputs)
            loss = self.loss_fn(out, target)
        loss.backward()
        if self.grad_clip is not None:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.grad_clip)
        self.optimizer.step()
        self.steps += 1
        return loss.detach()

    # -- checkpointing -----------------------------------------------------------
    def state_dict(self) -> dict:
        return {"model": self.model.module.state_dict(), "optimizer": self.optimizer.state_dict(),
                "reducer": self.state.state_dict() if self.state is not None else None, "steps": self.steps}

    def load_state_dict(self, d: dict) -> None:
        self.model.module.load_state_dict(d["model"])
        self.optimizer.load_state_dict(d["optimizer"])
        if self.state is not None and d.get("reducer") is not None:
            self.state.load_state_dict(d["reducer"], device=self.device)
        self.steps = d.get("steps", 0)

    def check(self) -> None:
        """Surface device-side communication errors (bounded waits that gave up)."""
        if self.state is not None:
            self.state.check_status()
