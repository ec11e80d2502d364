"""Count-sketch error compressors.

``DenseCS``       one hash row, fp32 storage    (reference: communication/compressors/CountSketch.py:102-182)
``HalfDenseCS``   one hash row, fp16 storage    (reference: communication/compressors/halfCountSketch.py:110-197)
``DenseCSHash3``  three hash rows, median query (reference: communication/compressors/CountSketchHash3.py:152-238)

A sketch keeps one row of width ``W = max(int(D * sketch_size), 1)`` per matrix
row.  Since the hash depends only on the column, the sketch is ``M @ H`` with a
sparse sign matrix ``H``; the column table is computed once per
``(D, W, seeds)`` and cached per device.

Differences from the reference, on purpose:
  * the hash seeds are part of ``state_dict()`` (the reference drops them, so a
    reloaded object could not be queried);
  * ``DenseCSHash3`` uses the same sign hash for its third row in query and
    update (the reference uses two different ones);
  * CPU tensors are supported (the library's host loops of ``csrc/cpu_ops.cu``, or
    PyTorch ops without the library); CUDA tensors run the sm_100a kernels of
    ``csrc/sketch.cu``.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..ops import native
from ..ops import reference as ref

_TABLE_CACHE: Dict[tuple, tuple] = {}


def default_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def tables_for(device, D: int, W: int, a: int, b: int, sign_offset=ref.SIGN_OFFSETS[0]):
    """(idx int64, sign fp32, packed int32, counts int32) on ``device``, cached."""
    device = torch.device(device)
    key = (device.type, device.index, D, W, a, b, tuple(sign_offset), ref.hash_layout())
    hit = _TABLE_CACHE.get(key)
    if hit is not None:
        return hit
    idx, sign = ref.hash_table(D, W, a, b, sign_offset, device="cpu")
    packed = torch.from_numpy(ref.packed_hash_table(D, W, a, b, sign_offset).copy())
    counts = torch.bincount(idx, minlength=W).to(torch.int32)
    out = (idx.to(device), sign.to(device), packed.to(device), counts.to(device))
    _TABLE_CACHE[key] = out
    return out


def block_csr_for(device, D: int, W: int, a: int, b: int, sign_offset=ref.SIGN_OFFSETS[0]):
    """The hash of ``(D, W)`` regrouped by cell block (``ops.reference.block_csr``) as an int32 tensor on
    ``device``, cached; ``None`` when this (D, W) uses the per-element hash."""
    device = torch.device(device)
    key = ("csr", device.type, device.index, D, W, a, b, tuple(sign_offset), ref.hash_layout())
    if key not in _TABLE_CACHE:
        csr = ref.block_csr(D, W, a, b, sign_offset)
        _TABLE_CACHE[key] = None if csr is None else torch.from_numpy(csr.copy()).to(device)
    return _TABLE_CACHE[key]


def _host_native(mat: torch.Tensor, cs: torch.Tensor) -> bool:
    """CPU tensors take the library's host loops (``csrc/cpu_ops.cu``: one pass per row, no index tensors)
    when it is built; ``CONEF_BACKEND=torch`` or a missing library leaves the PyTorch ops."""
    return (not mat.is_cuda and mat.dtype == torch.float32 and cs.dtype == torch.float32 and cs.is_contiguous()
            and os.environ.get("CONEF_BACKEND", "native") != "torch" and native.available())


class DenseCS:
    """Single-row count sketch of an ``(N, D)`` error matrix.

    ``query(t, alpha)``  : ``t += alpha * unsketch(cs)`` in place
    ``update(v, beta)``  : ``cs <- cs + sketch(v) - (1 - beta) * k_h * cs``
    ``clean(alpha)``     : ``cs *= alpha``
    """

    storage_dtype = torch.float32
    blk_size = 256

    def __init__(self, N: int, D: int, sketch_size: float, device=None, seed: int = 0,
                 storage: Optional[torch.Tensor] = None):
        self.N = int(N)
        self.D = int(D)
        self.range = ref.sketch_width(D, sketch_size)
        self.sketch_size = float(sketch_size)
        (self.a, self.b), = ref.derive_hash_seeds(seed, 1)
        device = torch.device(device) if device is not None else default_device()
        if storage is not None:
            assert storage.numel() == self.N * self.range and storage.dtype == self.storage_dtype
            self.cs = storage.view(self.N, self.range)
        else:
            self.cs = torch.zeros(self.N, self.range, dtype=self.storage_dtype, device=device)

    # -- numerics -----------------------------------------------------------
    def _tables(self):
        return tables_for(self.cs.device, self.D, self.range, self.a, self.b)

    def _check(self, t: torch.Tensor) -> torch.Tensor:
        if t.numel() != self.N * self.D:
            raise ValueError(f"expected {self.N}x{self.D} elements, got {tuple(t.shape)}")
        if t.device != self.cs.device:
            raise ValueError(f"sketch lives on {self.cs.device}, tensor on {t.device}")
        if not t.is_contiguous():
            raise ValueError("sketch operands must be contiguous")
        return t.view(self.N, self.D)

    def query(self, grad_plus_error: torch.Tensor, alpha: float) -> None:
        mat = self._check(grad_plus_error)
        idx, sign, packed, _ = self._tables()
        if native.use_native(mat) and mat.dtype == torch.float32 and self.cs.is_contiguous():
            native.check(native.lib().conef_sketch_query(
                mat.data_ptr(), self.cs.data_ptr(), int(self.cs.dtype == torch.float16), packed.data_ptr(),
                self.N, self.D, self.range, float(alpha), native.stream_ptr(mat.device)), "sketch_query")
        elif _host_native(mat, self.cs):
            native.lib().conef_cpu_sketch_query(mat.data_ptr(), self.cs.data_ptr(), packed.data_ptr(),
                                                self.N, self.D, self.range, float(alpha))
        else:
            ref.sketch_query_ref(mat, self.cs.float(), idx, sign, alpha)

    def update(self, vec: torch.Tensor, beta: float) -> None:
        mat = self._check(vec)
        idx, sign, packed, counts = self._tables()
        if native.use_native(mat) and mat.dtype == torch.float32 and self.cs.is_contiguous():
            native.check(native.lib().conef_sketch_update(
                mat.data_ptr(), self.cs.data_ptr(), int(self.cs.dtype == torch.float16), packed.data_ptr(),
                counts.data_ptr(), self.N, self.D, self.range, float(beta),
                native.stream_ptr(mat.device)), "sketch_update")
        elif _host_native(mat, self.cs):
            native.lib().conef_cpu_sketch_update(mat.data_ptr(), self.cs.data_ptr(), packed.data_ptr(),
                                                 counts.data_ptr(), self.N, self.D, self.range, float(beta))
        elif self.cs.dtype == torch.float32 and self.cs.is_contiguous():
            ref.sketch_update_ref(mat.float(), self.cs, idx, sign, beta)
        else:
            tmp = self.cs.float()
            ref.sketch_update_ref(mat.float(), tmp, idx, sign, beta)
            self.cs.copy_(tmp)

    def clean(self, alpha: float) -> None:
        self.cs.mul_(alpha)

    def nbytes(self) -> int:
        return self.cs.numel() * self.cs.element_size()

    # -- persistence ----------------------------------------------------------
    def state_dict(self) -> dict:
        return self.__getstate__()

    def load_state_dict(self, d: dict) -> None:
        self.__setstate__(d)

    def __getstate__(self) -> dict:
        return {"N": self.N, "D": self.D, "blk_size": self.blk_size, "range": self.range,
                "cs": self.cs.detach().cpu().numpy(), "a": self.a, "b": self.b,
                "sketch_size": self.sketch_size}

    def __setstate__(self, d: dict) -> None:
        keep = getattr(self, "cs", None)
        self.N, self.D, self.range = int(d["N"]), int(d["D"]), int(d["range"])
        self.a = int(d.get("a", ref.DEFAULT_A))
        self.b = int(d.get("b", ref.DEFAULT_B))
        self.sketch_size = float(d.get("sketch_size", self.range / max(self.D, 1)))
        cs = torch.from_numpy(np.asarray(d["cs"])).to(self.storage_dtype)
        if keep is not None and keep.numel() == cs.numel():
            keep.copy_(cs.reshape(keep.shape))  # keep arena-backed storage in place
            self.cs = keep
        else:
            self.cs = cs.to(default_device())

    def to(self, device) -> "DenseCS":
        self.cs = self.cs.to(device)
        return self


class HalfDenseCS(DenseCS):
    """Single-row sketch stored in fp16 (math in fp32): half the resting memory."""

    storage_dtype = torch.float16


class DenseCSHash3:
    """Three hash rows; query returns the median of the three estimates."""

    blk_size = 512

    def __init__(self, N: int, D: int, sketch_size: float, device=None, seed: int = 0,
                 split_budget: bool = False):
        self.N, self.D = int(N), int(D)
        width = sketch_size / 3.0 if split_budget else sketch_size
        self.range = ref.sketch_width(D, width)
        self.sketch_size = float(sketch_size)
        self.seeds = ref.derive_hash_seeds(seed, 3)
        device = torch.device(device) if device is not None else default_device()
        self.cs0 = torch.zeros(self.N, self.range, device=device)
        self.cs1 = torch.zeros(self.N, self.range, device=device)
        self.cs2 = torch.zeros(self.N, self.range, device=device)

    def _rows(self):
        return (self.cs0, self.cs1, self.cs2)

    def _tables(self):
        return [tables_for(self.cs0.device, self.D, self.range, a, b, off)
                for (a, b), off in zip(self.seeds, ref.SIGN_OFFSETS)]

    def _check(self, t):
        if t.numel() != self.N * self.D or not t.is_contiguous():
            raise ValueError("bad operand for DenseCSHash3")
        return t.view(self.N, self.D)

    def query(self, grad_plus_error: torch.Tensor, alpha: float) -> None:
        mat = self._check(grad_plus_error)
        tabs = self._tables()
        if native.use_native(mat) and mat.dtype == torch.float32:
            native.check(native.lib().conef_sketch3_query(
                mat.data_ptr(), self.cs0.data_ptr(), self.cs1.data_ptr(), self.cs2.data_ptr(),
                tabs[0][2].data_ptr(), tabs[1][2].data_ptr(), tabs[2][2].data_ptr(),
                self.N, self.D, self.range, float(alpha), native.stream_ptr(mat.device)), "sketch3_query")
        else:
            ref.sketch3_query_ref(mat, self._rows(), [(t[0], t[1]) for t in tabs], alpha)

    def update(self, vec: torch.Tensor, beta: float) -> None:
        mat = self._check(vec)
        tabs = self._tables()
        if native.use_native(mat) and mat.dtype == torch.float32:
            native.check(native.lib().conef_sketch3_update(
                mat.data_ptr(), self.cs0.data_ptr(), self.cs1.data_ptr(), self.cs2.data_ptr(),
                tabs[0][2].data_ptr(), tabs[1][2].data_ptr(), tabs[2][2].data_ptr(),
                self.N, self.D, self.range, float(beta), native.stream_ptr(mat.device)), "sketch3_update")
        else:
            ref.sketch3_update_ref(mat, self._rows(), [(t[0], t[1]) for t in tabs], beta)

    def clean(self, alpha: float) -> None:
        for cs in self._rows():
            cs.mul_(alpha)

    def nbytes(self) -> int:
        return sum(cs.numel() * cs.element_size() for cs in self._rows())

    def state_dict(self) -> dict:
        return self.__getstate__()

    def load_state_dict(self, d: dict) -> None:
        self.__setstate__(d)

    def __getstate__(self) -> dict:
        return {"N": self.N, "D": self.D, "blk_size": self.blk_size, "range": self.range,
                "cs0": self.cs0.detach().cpu().numpy(), "cs1": self.cs1.detach().cpu().numpy(),
                "cs2": self.cs2.detach().cpu().numpy(), "seeds": [list(s) for s in self.seeds],
                "sketch_size": self.sketch_size}

    def __setstate__(self, d: dict) -> None:
        self.N, self.D, self.range = int(d["N"]), int(d["D"]), int(d["range"])
        self.sketch_size = float(d.get("sketch_size", 0.0))
        self.seeds = [tuple(s) for s in d.get("seeds", list(zip(ref.HASH3_A, ref.HASH3_B)))]
        dev = default_device()
        self.cs0 = torch.from_numpy(np.asarray(d["cs0"])).float().to(dev)
        self.cs1 = torch.from_numpy(np.asarray(d["cs1"])).float().to(dev)
        self.cs2 = torch.from_numpy(np.asarray(d["cs2"])).float().to(dev)

    def to(self, device) -> "DenseCSHash3":
        self.cs0, self.cs1, self.cs2 = (c.to(device) for c in self._rows())
        return self
