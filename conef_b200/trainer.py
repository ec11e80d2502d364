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


def _graph_submodules(model, modules, sample_inputs, device, autocast_dtype, channels_last) -> int:
    """Capture forward and backward of ``modules`` as CUDA graphs (``torch.cuda.make_graphed_callables``; must
    happen before the model is wrapped in DistributedDataParallel).  The input shapes come from one dry run
    of the model on ``sample_inputs``; a module called with another shape, without gradients or in
    evaluation mode runs its own code.  Returns the number of modules captured."""
    if not modules:
        return 0
    sample = []
    for t in sample_inputs:
        t = t.to(device)
        if channels_last and t.dim() == 4:
            t = t.contiguous(memory_format=torch.channels_last)
        sample.append(t)
    shapes, handles = {}, []
    def note_shape(mod, args):      # (a pre-hook's return value would replace the inputs: return nothing)
        shapes.setdefault(id(mod), (tuple(args[0].shape), args[0].dtype, len(args)))

    for m in modules:
        handles.append(m.register_forward_pre_hook(note_shape))
    ctx = (lambda: torch.autocast("cuda", dtype=autocast_dtype, cache_enabled=False)) if autocast_dtype is not None \
        else contextlib.nullcontext
    was_training = model.training
    buffers = {name: b.detach().clone() for name, b in model.named_buffers()}      # batch-norm statistics, counters
    model.train()
    with torch.no_grad(), ctx():
        model(*sample)
    for h in handles:
        h.remove()
    if any(id(m) not in shapes or shapes[id(m)][2] != 1 for m in modules):
        with torch.no_grad():
            for name, b in model.named_buffers():
                b.copy_(buffers[name])
        model.train(was_training)
        return 0
    args = []
    for m in modules:
        shape, dtype, _ = shapes[id(m)]
        x = torch.randn(shape, device=device, dtype=dtype)
        if channels_last and x.dim() == 4:
            x = x.contiguous(memory_format=torch.channels_last)
        args.append((x.requires_grad_(True),))
    eager = [m.forward for m in modules]
    with ctx():
        torch.cuda.make_graphed_callables(tuple(modules), tuple(args), num_warmup_iters=3)
    # the warm-up ran on a side stream, so the parameters' AccumulateGrad nodes belong to that stream: autograd
    # orders them against the training stream with an event and says so at every backward pass
    mute = getattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch", None)
    if mute is not None:
        mute(False)
    for m, own, (shape, dtype, _) in zip(modules, eager, (shapes[id(m)] for m in modules)):
        graphed = m.forward

        def guarded(x, _g=graphed, _own=own, _shape=shape, _dtype=dtype):
            if torch.is_grad_enabled() and x.requires_grad and tuple(x.shape) == _shape and x.dtype == _dtype:
                return _g(x)
            return _own(x)
        m.forward = guarded
    with torch.no_grad():      # in place: the graphs hold the buffers' addresses
        for name, b in model.named_buffers():
            b.copy_(buffers[name])
    model.train(was_training)
    return len(modules)


class DataParallelTrainer:
    def __init__(self, model: torch.nn.Module, optimizer_factory: Callable, loss_fn: Callable, *,
                 reducer: Union[None, Any, Tuple[Any, Callable]] = None, device: Optional[torch.device] = None,
                 autocast_dtype: Optional[torch.dtype] = None, bucket_cap_mb: float = 25.0,
                 channels_last: bool = False, grad_clip: Optional[float] = None,
                 forward_fn: Optional[Callable] = None,
                 graph_modules: Optional[Callable[[torch.nn.Module], Sequence[torch.nn.Module]]] = None,
                 graph_sample_inputs: Optional[Sequence[torch.Tensor]] = None,
                 cudnn_autotune: bool = False):
        """``reducer`` is ``None`` (plain all-reduce), an argparse-like namespace with
        ``grad_reducer`` etc. (see :func:`conef_b200.get_comm_hooks`), or a ``(state, hook)`` pair.
        ``optimizer_factory(params)`` builds the optimizer on the wrapped model's parameters.
        ``forward_fn(model, *inputs)`` customises the forward call (default ``model(*inputs)``).
        ``graph_modules(model)`` names submodules (each taking and returning one tensor) whose forward and
        backward passes are captured as CUDA graphs from ``graph_sample_inputs`` (one batch of model inputs
        of the training shape): a step of a deep CNN is otherwise bound by the host's launch rate, not by
        the GPU.  Other input shapes, evaluation mode and CPU runs go through the modules' own code.
        ``cudnn_autotune`` lets cuDNN time its convolution engines on the first call of every shape and keep
        the fastest (``torch.backends.cudnn.benchmark``, a process-wide switch; for fixed-shape CNN training)."""
        if cudnn_autotune and torch.cuda.is_available():
            torch.backends.cudnn.benchmark = True
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
                else torch.device("cpu")
        self.device = device
        model = model.to(device)
        if channels_last:
            model = model.to(memory_format=torch.channels_last)
        self.channels_last = channels_last
        self.graphed_modules = 0
        if graph_modules is not None and graph_sample_inputs is not None and device.type == "cuda":
            self.graphed_modules = _graph_submodules(model, list(graph_modules(model)), graph_sample_inputs, device,
                                                     autocast_dtype, channels_last)
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
