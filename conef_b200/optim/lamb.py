"""LAMB optimizer with a multi-tensor CUDA implementation.

Stands in for ``apex.optimizers.FusedLAMB`` that the reference's BERT driver
uses (examples/BertPretraining/run_pretraining_conef.py:42,449-450): global
gradient-norm clipping, Adam moments with bias correction, decoupled weight
decay inside the update direction, and a per-tensor trust ratio
``|w| / |update|``.

On CUDA fp32 parameters the whole step is three grouped kernel launches over
all tensors (``csrc/lamb.cu``); the gradient buffers are overwritten with the
update direction, as apex does.  On CPU (or other dtypes) the same math runs as
PyTorch ops.
"""
from __future__ import annotations

import math
from typing import List

import numpy as np
import torch
from torch.optim import Optimizer

from ..ops import native
from ..ops.reference import lamb_step_ref

CHUNK = 65536


class FusedLAMB(Optimizer):
    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01,
                 max_grad_norm=1.0, grad_scale=1.0):
        defaults = dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay,
                        max_grad_norm=max_grad_norm)
        super().__init__(params, defaults)
        self.grad_scale = grad_scale
        self._tables = {}

    def _init_state(self, p):
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return st

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        # global gradient norm over every parameter of every group (apex semantics)
        all_params = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not all_params:
            return loss
        fused = all(p.is_cuda and p.dtype == torch.float32 and p.grad.dtype == torch.float32
                    and p.is_contiguous() and p.grad.is_contiguous() for p in all_params) \
            and native.use_native(all_params[0])
        if fused:
            self._step_fused()
        else:
            self._step_torch(all_params)
        return loss

    # -- PyTorch ops -------------------------------------------------------------
    def _step_torch(self, all_params):
        max_norm = self.param_groups[0]["max_grad_norm"]
        gmul = 1.0 / self.grad_scale
        if max_norm and max_norm > 0:
            total = math.sqrt(sum(float(p.grad.float().pow(2).sum()) for p in all_params)) * gmul
            if total > max_norm:
                gmul *= max_norm / total
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._init_state(p)
                st["step"] += 1
                lamb_step_ref(p, p.grad * gmul, st["exp_avg"], st["exp_avg_sq"], group["lr"], b1, b2, group["eps"],
                              group["weight_decay"], st["step"], 1.0, group["bias_correction"])

    # -- grouped CUDA kernels ------------------------------------------------------
    def _uniform_groups(self) -> bool:
        """One launch set covers all groups when they differ only in weight decay."""
        keys = ("lr", "betas", "eps", "bias_correction", "max_grad_norm")
        first = self.param_groups[0]
        return all(all(g[k] == first[k] for k in keys) for g in self.param_groups)

    def _step_fused(self):
        lib = native.lib()
        if not self._uniform_groups():
            return self._step_torch([p for g in self.param_groups for p in g["params"] if p.grad is not None])
        entries = [(p, g["weight_decay"]) for g in self.param_groups for p in g["params"] if p.grad is not None]
        params = [p for p, _ in entries]
        for p in params:
            self._init_state(p)
        key = tuple((p.data_ptr(), p.grad.data_ptr(), wd) for p, wd in entries)
        tab = self._tables.get("all")
        if tab is None or tab["key"] != key:
            rec = np.zeros(len(params), dtype=native.LAMB_DTYPE)
            chunks = []
            for t, (p, wd) in enumerate(entries):
                st = self.state[p]
                rec[t] = (p.data_ptr(), p.grad.data_ptr(), st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(),
                          p.numel(), wd, 0)
                chunks += [(t, c) for c in range((p.numel() + CHUNK - 1) // CHUNK)]
            dev = params[0].device
            tab = {"key": key, "tensors": native.upload_struct_array(rec, dev),
                   "chunks": torch.from_numpy(np.asarray(chunks, dtype=np.int32)).to(dev),
                   "nchunks": len(chunks), "norms": torch.zeros(1 + 2 * len(params), device=dev),
                   "n": len(params)}
            self._tables["all"] = tab
        step = self.state[params[0]]["step"] + 1
        for p in params:
            self.state[p]["step"] = step
        group = self.param_groups[0]
        b1, b2 = group["betas"]
        native.check(lib.conef_lamb_step(
            tab["tensors"].data_ptr(), tab["n"], tab["chunks"].data_ptr(), tab["nchunks"], CHUNK,
            tab["norms"].data_ptr(), float(group["lr"]), float(b1), float(b2), float(group["eps"]), int(step),
            int(bool(group["bias_correction"])), float(self.grad_scale), float(group["max_grad_norm"] or 0.0),
            native.stream_ptr(params[0].device)), "lamb_step")
