"""SGD with momentum as one multi-tensor CUDA launch.

``torch.optim.SGD`` semantics (weight decay added to the gradient, momentum buffer initialised with the
first gradient, dampening, Nesterov), for the image-classification and language-modelling drivers of the
reference (examples/ImageClassification/main.py:188-190, examples/LanguageModeling/main.py).  On CUDA fp32
parameters the step is a single pass over parameters, gradients and momentum buffers
(``csrc/lamb.cu:k_sgd_step``); PyTorch's foreach path is about fifteen launches and three passes.  The
kernel walks the storage, so a parameter qualifies when it is dense in any dimension order (contiguous or
channels-last) and its gradient and momentum buffer have the same strides; the others of a group (CPU,
other dtypes, strided views) run as PyTorch ops beside it.  ``zero_grad(set_to_none=False)`` clears all
gradients with one multi-tensor call, which keeps the gradient addresses (and the kernel's tensor table)
stable from step to step.
"""
from __future__ import annotations

import numpy as np
import torch
from torch.optim import Optimizer

from ..ops import native

CHUNK = 65536


def _dense(t):
    """Non-overlapping and dense: the elements fill the storage range in some dimension order."""
    if t.is_contiguous():
        return True
    if t.dim() == 4:
        return t.is_contiguous(memory_format=torch.channels_last)
    if t.dim() == 5:
        return t.is_contiguous(memory_format=torch.channels_last_3d)
    return False


def _fusable(p):
    g = p.grad
    return (p.is_cuda and p.dtype == torch.float32 and g.dtype == torch.float32 and g.layout == torch.strided
            and _dense(p) and g.stride() == p.stride())


class FusedSGD(Optimizer):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        defaults = dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay, nesterov=nesterov)
        super().__init__(params, defaults)
        self._tables = {}

    def _buf(self, p):
        st = self.state[p]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = None
        return st

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for gi, group in enumerate(self.param_groups):
            params = [p for p in group["params"] if p.grad is not None]
            if not params:
                continue
            fused = [p for p in params if _fusable(p)]
            if fused and not native.use_native(fused[0]):
                fused = []
            if len(fused) != len(params):
                chosen = set(map(id, fused))
                self._step_torch(group, [p for p in params if id(p) not in chosen])
            if fused:
                self._step_fused(gi, group, fused)
        return loss

    @torch.no_grad()
    def zero_grad(self, set_to_none: bool = True):
        if set_to_none:
            return super().zero_grad(set_to_none=True)
        by_kind = {}
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    if p.grad.grad_fn is not None:
                        p.grad.detach_()
                    else:
                        p.grad.requires_grad_(False)
                    by_kind.setdefault((p.grad.device, p.grad.dtype), []).append(p.grad)
        for grads in by_kind.values():
            torch._foreach_zero_(grads)

    def _step_torch(self, group, params):
        lr, mu, damp, wd, nest = (group[k] for k in ("lr", "momentum", "dampening", "weight_decay", "nesterov"))
        for p in params:
            g = p.grad
            if wd != 0:
                g = g.add(p, alpha=wd)
            if mu != 0:
                st = self._buf(p)
                if st["momentum_buffer"] is None:
                    st["momentum_buffer"] = g.clone()
                else:
                    st["momentum_buffer"].mul_(mu).add_(g, alpha=1 - damp)
                g = g.add(st["momentum_buffer"], alpha=mu) if nest else st["momentum_buffer"]
            p.add_(g, alpha=-lr)

    def _step_fused(self, gi, group, params):
        lr, mu, damp, wd, nest = (group[k] for k in ("lr", "momentum", "dampening", "weight_decay", "nesterov"))
        first = False
        if mu != 0:
            fresh = [self._buf(p)["momentum_buffer"] is None for p in params]
            if any(fresh) and not all(fresh):      # parameters that joined later: one step through the PyTorch ops
                return self._step_torch(group, params)
            first = all(fresh)
            if first:
                for p in params:
                    self.state[p]["momentum_buffer"] = torch.empty_like(p, memory_format=torch.preserve_format)
            for p in params:       # a buffer restored from a checkpoint of another memory format: re-lay it once
                buf = self.state[p]["momentum_buffer"]
                if buf.stride() != p.stride() or buf.dtype != p.dtype or buf.device != p.device:
                    self.state[p]["momentum_buffer"] = torch.empty_like(p, memory_format=torch.preserve_format).copy_(buf)
        key = tuple((p.data_ptr(), p.grad.data_ptr(), self.state[p]['momentum_buffer'].data_ptr() if mu != 0 else 0)
                    for p in params) + (wd,)
        tab = self._tables.get(gi)
        if tab is None or tab["key"] != key:
            rec = np.zeros(len(params), dtype=native.LAMB_DTYPE)
            chunks = []
            for t, p in enumerate(params):
                m = self.state[p]["momentum_buffer"].data_ptr() if mu != 0 else 0
                rec[t] = (p.data_ptr(), p.grad.data_ptr(), m, 0, p.numel(), wd, 0)
                chunks += [(t, c) for c in range((p.numel() + CHUNK - 1) // CHUNK)]
            dev = params[0].device
            tab = {"key": key, "tensors": native.upload_struct_array(rec, dev),
                   "chunks": torch.from_numpy(np.asarray(chunks, dtype=np.int32)).to(dev), "nchunks": len(chunks),
                   "n": len(params)}
            self._tables[gi] = tab
        native.check(native.lib().conef_sgd_step(
            tab["tensors"].data_ptr(), tab["n"], tab["chunks"].data_ptr(), tab["nchunks"], CHUNK, float(lr), float(mu),
            float(damp), int(bool(nest)), int(first), native.stream_ptr(params[0].device)), "sgd_step")
