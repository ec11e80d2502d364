"""Error compressors that have no counterpart in the reference's compressor
directory: dense storage (classic error feedback), top-k (the reference keeps
this inline in communication/hPowerSGD_hook.py:90-97), 8-bit group
quantisation and low-rank factors.

All of them follow the contract of the count sketches:

``query(t, alpha)``   ``t += alpha * e_hat``                       (in place)
``update(v, beta)``   ``e_hat <- C(beta * e_hat + v)``             (C = the compressor)

With ``alpha = 1 - beta`` only that fraction of the remembered error is fed
back each step and the rest stays in memory; ``beta = 0`` is classic error
feedback with a compressed store.
"""
from __future__ import annotations

import numpy as np
import torch

from ..ops import native
from ..ops import reference as ref
from .count_sketch import default_device


class _Base:
    def state_dict(self) -> dict:
        return self.__getstate__()

    def load_state_dict(self, d: dict) -> None:
        self.__setstate__(d)


class DenseError(_Base):
    """Uncompressed error buffer of shape ``(N, D)``."""

    def __init__(self, N, D, device=None, storage=None):
        self.N, self.D = int(N), int(D)
        device = torch.device(device) if device is not None else default_device()
        self.err = storage.view(N, D) if storage is not None else torch.zeros(N, D, device=device)

    def query(self, t, alpha):
        t.view(self.N, self.D).add_(self.err, alpha=alpha)

    def update(self, v, beta):
        self.err.mul_(beta).add_(v.view(self.N, self.D))

    def clean(self, alpha):
        self.err.mul_(alpha)

    def nbytes(self):
        return self.err.numel() * self.err.element_size()

    def __getstate__(self):
        return {"N": self.N, "D": self.D, "err": self.err.detach().cpu().numpy()}

    def __setstate__(self, d):
        self.N, self.D = int(d["N"]), int(d["D"])
        self.err = torch.from_numpy(np.asarray(d["err"])).to(default_device())


class TopKError(DenseError):
    """Keeps the ``max(1, int(0.5 * ratio * numel))`` largest-magnitude entries.

    Stored dense-with-zeros, exactly as the reference does "for simulation"
    (communication/hPowerSGD_hook.py:90-97); ``nbytes`` reports what a packed
    (value, index) store of the kept entries would need.
    """

    def __init__(self, N, D, topk_ratio=0.4, device=None):
        super().__init__(N, D, device)
        self.topk_ratio = float(topk_ratio)

    def update(self, v, beta):
        self.err.mul_(beta).add_(v.view(self.N, self.D))
        if native.use_native(self.err) and self.err.dtype == torch.float32 and self.err.is_contiguous():
            self._native_keep()
        else:
            ref.topk_keep_(self.err, self.topk_ratio)

    def _native_keep(self):
        """Radix select on the device (csrc/topk.cu) instead of a sort."""
        lib = native.lib()
        tabs = getattr(self, "_tk", None)
        if tabs is None or tabs[0].device != self.err.device:
            rec = np.zeros(1, dtype=native.MAT_DTYPE)
            rec[0]["n"], rec[0]["m"] = self.N, self.D
            ch = lib.conef_topk_chunk()
            nt = (self.N * self.D + ch - 1) // ch
            tiles = np.zeros((nt, 2), dtype=np.int32)
            tiles[:, 1] = np.arange(nt)
            dev = self.err.device
            tabs = (native.upload_struct_array(rec, dev), torch.from_numpy(tiles).to(dev),
                    torch.zeros(2050, dtype=torch.int32, device=dev), nt)
            self._tk = tabs
        native.check(lib.conef_topk_keep(tabs[0].data_ptr(), 1, tabs[1].data_ptr(), tabs[3], self.err.data_ptr(),
                                         self.topk_ratio, tabs[2].data_ptr(), native.stream_ptr(self.err.device)),
                     "topk_keep")

    def nbytes(self):
        return max(1, int(0.5 * self.topk_ratio * self.N * self.D)) * 8

    def __getstate__(self):
        d = super().__getstate__()          # the device tables (_tk) are rebuilt on demand
        d["topk_ratio"] = self.topk_ratio
        return d

    def __setstate__(self, d):
        super().__setstate__(d)
        self.topk_ratio = float(d.get("topk_ratio", 0.4))


class Quant8Error(_Base):
    """Symmetric int8 codes with one fp32 scale per 256 consecutive elements."""

    GROUP = ref.QUANT_GROUP

    def __init__(self, N, D, device=None, codes=None, scales=None):
        self.N, self.D = int(N), int(D)
        n = self.N * self.D
        device = torch.device(device) if device is not None else default_device()
        groups = (n + self.GROUP - 1) // self.GROUP
        self.codes = codes if codes is not None else torch.zeros(n, dtype=torch.int8, device=device)
        self.scales = scales if scales is not None else torch.zeros(groups, dtype=torch.float32, device=device)

    def _flat(self, t):
        if t.numel() != self.N * self.D or not t.is_contiguous():
            raise ValueError("bad operand for Quant8Error")
        return t.view(-1)

    def query(self, t, alpha):
        flat = self._flat(t)
        if native.use_native(flat) and flat.dtype == torch.float32:
            native.check(native.lib().conef_quant8_query(
                flat.data_ptr(), self.codes.data_ptr(), self.scales.data_ptr(), flat.numel(), float(alpha),
                native.stream_ptr(flat.device)), "quant8_query")
        else:
            flat.add_(ref.quant8_decode_ref(self.codes, self.scales), alpha=alpha)

    def update(self, v, beta):
        flat = self._flat(v)
        if native.use_native(flat) and flat.dtype == torch.float32:
            native.check(native.lib().conef_quant8_update(
                flat.data_ptr(), self.codes.data_ptr(), self.scales.data_ptr(), flat.numel(), float(beta),
                native.stream_ptr(flat.device)), "quant8_update")
        else:
            keep = ref.quant8_decode_ref(self.codes, self.scales) * beta + flat.float()
            codes, scales = ref.quant8_encode_ref(keep)
            self.codes.copy_(codes)
            self.scales.copy_(scales)

    def clean(self, alpha):
        self.scales.mul_(alpha)

    def nbytes(self):
        return self.codes.numel() + self.scales.numel() * 4

    def __getstate__(self):
        return {"N": self.N, "D": self.D, "codes": self.codes.detach().cpu().numpy(),
                "scales": self.scales.detach().cpu().numpy()}

    def __setstate__(self, d):
        self.N, self.D = int(d["N"]), int(d["D"])
        dev = default_device()
        codes = torch.from_numpy(np.asarray(d["codes"]))
        scales = torch.from_numpy(np.asarray(d["scales"]))
        if getattr(self, "codes", None) is not None and self.codes.numel() == codes.numel():
            self.codes.copy_(codes)
            self.scales.copy_(scales)
        else:
            self.codes, self.scales = codes.to(dev), scales.to(dev)


class LowRankError(_Base):
    """Rank-``k`` factors ``U (N x k)``, ``V (D x k)`` with ``e_hat = U V^T``.

    ``update`` runs one warm-started power-iteration step on
    ``T = beta * U V^T + v`` without ever forming ``T``:
    ``U' = orth(T V)``, ``V' = T^T U'`` — two tall-skinny products of the same
    shape as PowerSGD's own, so the same kernels serve both.
    """

    def __init__(self, N, D, rank=4, device=None, seed=0):
        self.N, self.D = int(N), int(D)
        self.rank = int(min(rank, N, D))
        device = torch.device(device) if device is not None else default_device()
        gen = torch.Generator().manual_seed(1234 + seed)
        self.U = torch.zeros(self.N, self.rank, device=device)
        self.V = torch.randn(self.D, self.rank, generator=gen).to(device)
        ref.gram_schmidt_ref(self.V)

    def query(self, t, alpha):
        t.view(self.N, self.D).addmm_(self.U, self.V.t(), alpha=alpha)

    def update(self, v, beta):
        v = v.view(self.N, self.D)
        # T V = beta * U (V^T V) + v V
        tv = v @ self.V
        if beta != 0:
            tv.add_(self.U @ (self.V.t() @ self.V), alpha=beta)
        # columns that collapsed to zero (first steps) would give NaN in Gram-Schmidt
        ref.gram_schmidt_ref(tv, eps=1e-12)
        new_v = v.t() @ tv
        if beta != 0:
            new_v.add_(self.V @ (self.U.t() @ tv), alpha=beta)
        self.U, self.V = tv, new_v

    def clean(self, alpha):
        self.U.mul_(alpha)

    def nbytes(self):
        return (self.U.numel() + self.V.numel()) * 4

    def __getstate__(self):
        return {"N": self.N, "D": self.D, "rank": self.rank, "U": self.U.detach().cpu().numpy(),
                "V": self.V.detach().cpu().numpy()}

    def __setstate__(self, d):
        self.N, self.D, self.rank = int(d["N"]), int(d["D"]), int(d["rank"])
        dev = default_device()
        self.U = torch.from_numpy(np.asarray(d["U"])).to(dev)
        self.V = torch.from_numpy(np.asarray(d["V"])).to(dev)


ERROR_COMPRESSORS = ("count_sketch", "count_sketch3", "half_count_sketch", "topk", "quant8", "lowrank", "dense")


def make_error_compressor(kind: str, N: int, D: int, *, sketch_size: float = 0.5, seed: int = 0,
                          topk_ratio: float = 0.4, rank: int = 4, device=None):
    """Factory used by the hooks; ``kind`` is one of :data:`ERROR_COMPRESSORS`."""
    from .count_sketch import DenseCS, DenseCSHash3, HalfDenseCS

    if kind == "count_sketch":
        return DenseCS(N, D, sketch_size, device=device, seed=seed)
    if kind == "half_count_sketch":
        return HalfDenseCS(N, D, sketch_size, device=device, seed=seed)
    if kind == "count_sketch3":
        return DenseCSHash3(N, D, sketch_size, device=device, seed=seed)
    if kind == "topk":
        return TopKError(N, D, topk_ratio, device=device)
    if kind == "quant8":
        return Quant8Error(N, D, device=device)
    if kind == "lowrank":
        return LowRankError(N, D, rank, device=device, seed=seed)
    if kind == "dense":
        return DenseError(N, D, device=device)
    raise ValueError(f"unknown error compressor {kind!r}; choose from {ERROR_COMPRESSORS}")
