"""Per-bucket execution plans.

DDP hands a hook one flat gradient bucket plus the list of per-parameter
gradient views.  The reference re-derives the partition into "compress" and
"keep uncompressed" tensors, and all offsets, in Python loops on every call
(communication/powerSGD_hook.py:386-471, communication/RandomBlock_hook.py:170-209).
Here that work is done once per bucket layout and frozen into a
:class:`BucketPlan`; the native engine turns the plan into device-resident
descriptor tables so that every step is a handful of grouped kernel launches.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import torch

from ..ops.reference import should_compress


@dataclass
class MatEntry:
    """A tensor compressed as an ``(n, m)`` matrix."""
    g_off: int       # element offset inside the bucket
    n: int
    m: int
    r: int
    p_off: int       # offset of the (n, r) block in the flat P memory
    q_off: int       # offset of the (m, r) block in the flat Q memory
    index: int       # position among the bucket's gradients

    @property
    def numel(self) -> int:
        return self.n * self.m


@dataclass
class SegEntry:
    """A tensor sent uncompressed."""
    g_off: int
    numel: int
    dst_off: int     # offset inside the staging buffer
    index: int


@dataclass
class BucketPlan:
    signature: tuple
    total: int
    mats: List[MatEntry] = field(default_factory=list)
    segs: List[SegEntry] = field(default_factory=list)
    total_p: int = 0
    total_q: int = 0
    total_unc: int = 0
    numel_before: int = 0
    numel_after: int = 0

    @property
    def max_rank(self) -> int:
        return max((e.r for e in self.mats), default=0)


def bucket_signature(buffer: torch.Tensor, grads: Sequence[torch.Tensor]) -> tuple:
    return (buffer.numel(), str(buffer.device), buffer.dtype, tuple(tuple(g.shape) for g in grads))


def grad_offsets(buffer: torch.Tensor, grads: Sequence[torch.Tensor]) -> List[int]:
    """Element offset of every gradient view inside the bucket buffer."""
    base = buffer.data_ptr()
    esz = buffer.element_size()
    offs = []
    running = 0
    for g in grads:
        if g.numel() == 0:
            offs.append(running)
            continue
        off = (g.data_ptr() - base) // esz
        dense = g.is_contiguous() or (g.dim() == 4 and g.is_contiguous(memory_format=torch.channels_last))
        if off < 0 or off + g.numel() > buffer.numel() or not dense:
            # not a dense view of the buffer (should not happen with DDP): assume packed order
            off = running
        offs.append(off)
        running = off + g.numel()
    return offs


def build_powersgd_plan(buffer: torch.Tensor, grads: Sequence[torch.Tensor], rank: int,
                        min_compression_rate: float) -> BucketPlan:
    """Partition as in communication/powerSGD_hook.py:394-418 of the reference."""
    # A gradient is viewed as (shape[0], numel / shape[0]) over its chunk of the bucket *as it
    # lies in memory*.  For channels-last convolution weights the chunk is ordered
    # (out, kh, kw, in): still one row per output channel, with the columns permuted - which
    # changes neither the low-rank structure nor the statistics of the sketch.
    plan = BucketPlan(signature=bucket_signature(buffer, grads), total=buffer.numel())
    offs = grad_offsets(buffer, grads)
    for i, (g, off) in enumerate(zip(grads, offs)):
        if g.dim() == 0 or g.numel() == 0:
            n, m = 1, g.numel()
        else:
            n = g.shape[0]
            m = g.numel() // max(n, 1)
        r = min(n, m, rank)
        ok, before, after = should_compress(n, m, r, min_compression_rate) if g.numel() else (False, 0, 0)
        plan.numel_before += before
        if ok:
            plan.mats.append(MatEntry(off, n, m, r, plan.total_p, plan.total_q, i))
            plan.total_p += n * r
            plan.total_q += m * r
            plan.numel_after += after
        else:
            plan.segs.append(SegEntry(off, g.numel(), plan.total_unc, i))
            plan.total_unc += g.numel()
            plan.numel_after += before
    return plan


def build_batched_plan(total_length: int, rank: int, device, dtype) -> Tuple[BucketPlan, int]:
    """One zero-padded square matrix per bucket (communication/powerSGD_hook.py:656-663)."""
    side = math.ceil(math.sqrt(total_length))
    plan = BucketPlan(signature=("batched", total_length, str(device), dtype), total=side * side)
    r = min(side, rank)
    plan.mats.append(MatEntry(0, side, side, r, 0, 0, 0))
    plan.total_p = side * r
    plan.total_q = side * r
    plan.numel_before = total_length
    plan.numel_after = side * rank * 2
    return plan, side


@dataclass
class BlockEntry:
    """A tensor handled by the random-block compressor, viewed as ``(n, m)``."""
    g_off: int
    n: int
    m: int
    block: int
    stage_off: int
    index: int

    @property
    def numel(self) -> int:
        return self.n * self.m


@dataclass
class BlockPlan:
    signature: tuple
    total: int
    blocks: List[BlockEntry] = field(default_factory=list)
    segs: List[SegEntry] = field(default_factory=list)
    total_block: int = 0
    total_unc: int = 0


def build_block_plan(buffer: torch.Tensor, grads: Sequence[torch.Tensor], ratio: float) -> BlockPlan:
    """Partition as in communication/RandomBlock_hook.py:170-209: tensors with
    two or more dimensions send one contiguous block of
    ``max(1, int(ratio * numel))`` elements, the rest go uncompressed."""
    plan = BlockPlan(signature=bucket_signature(buffer, grads) + (ratio,), total=buffer.numel())
    offs = grad_offsets(buffer, grads)
    for i, (g, off) in enumerate(zip(grads, offs)):
        if g.dim() <= 1 or g.numel() == 0:
            plan.segs.append(SegEntry(off, g.numel(), plan.total_unc, i))
            plan.total_unc += g.numel()
        else:
            n = g.shape[0]
            m = g.numel() // n
            block = max(1, int(ratio * g.numel()))
            plan.blocks.append(BlockEntry(off, n, m, block, plan.total_block, i))
            plan.total_block += block
    return plan
