"""Symmetric (peer-addressable) device buffers for in-kernel collectives.

One :class:`SymmBuffer` is a same-sized allocation on every rank of a process
group whose device pointers are known to all ranks, so that a kernel on one
GPU can load from / store to the peers' copies over NVLink.  Layout of each
rank's allocation::

    [ flags: 64 x uint32 ][ region 0, slot 0 ][ region 1, slot 0 ] ... [ region 0, slot 1 ] ...

Regions are sized by the caller (e.g. staging / P / Q of one bucket) and are
double-buffered: step ``s`` uses slot ``s % 2`` so that a rank running one
phase ahead never overwrites data a slower peer is still reading.

Backends, tried in order unless ``CONEF_COMM`` pins one:
  * ``symm`` — ``torch.distributed._symmetric_memory`` (CUDA VMM handles);
  * ``ipc``  — a dedicated ``cudaMalloc`` exported with legacy CUDA IPC handles
    that are exchanged through the process group;
and when neither works the hooks use NCCL collectives instead.

Only plain peer loads/stores are issued on these buffers; they are never the
source of a TMA or cluster-multicast load.
"""
from __future__ import annotations

import ctypes as C
import logging
import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import native

logger = logging.getLogger(__name__)

FLAG_WORDS = 64
FLAG_BYTES = FLAG_WORDS * 4
ALIGN = 256

# Bound on device-side polling of a peer flag.  Each poll sleeps ~64 ns plus the
# NVLink round trip, so this is on the order of a couple of seconds.
DEFAULT_SPIN_LIMIT = int(os.environ.get("CONEF_SPIN_LIMIT", 4_000_000))


class SymmUnavailable(RuntimeError):
    pass


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class SymmBuffer:
    def __init__(self, region_floats: Sequence[int], group, device: torch.device, backend: str = "auto"):
        self.group = group
        self.device = device
        self.world = group.size()
        self.rank = dist.get_rank(group)
        self.region_floats = list(region_floats)
        # byte offsets of every (slot, region)
        self.offsets: List[List[int]] = []
        cursor = _round_up(FLAG_BYTES, ALIGN)
        for _slot in range(2):
            row = []
            for nf in self.region_floats:
                row.append(cursor)
                cursor = _round_up(cursor + nf * 4, ALIGN)
            self.offsets.append(row)
        self.total_bytes = cursor
        self._ipc_ptrs: List[int] = []
        self._handle = None
        self.backend = None
        errors = []
        order = {"auto": ("symm", "ipc"), "symm": ("symm",), "ipc": ("ipc",)}[backend]
        for name in order:
            try:
                getattr(self, f"_init_{name}")()
                self.backend = name
                break
            except Exception as exc:  # noqa: BLE001 - any failure means "try the next backend"
                errors.append(f"{name}: {type(exc).__name__}: {exc}")
        # every rank must agree, otherwise some would wait on flags nobody writes
        ok = torch.tensor([1 if self.backend else 0], device=device, dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            raise SymmUnavailable("; ".join(errors) or "a peer could not set up symmetric memory")
        self._build_pointer_tables()
        # flags start at zero everywhere before anyone may signal; the regions start at zero because
        # the fused pipeline accumulates into them and only clears a slot after it has been read
        self.local_bytes.zero_()
        torch.cuda.current_stream(device).synchronize()
        dist.barrier(group=group)

    # -- backends ------------------------------------------------------------
    def _init_symm(self):
        import torch.distributed._symmetric_memory as symm_mem

        t = symm_mem.empty(self.total_bytes, dtype=torch.uint8, device=self.device)
        hdl = symm_mem.rendezvous(t, group=self.group)
        self.local_bytes = t
        self._handle = hdl
        self.base_ptrs = [int(p) for p in hdl.buffer_ptrs]

    def _init_ipc(self):
        lib = native.lib()
        cudart = C.CDLL("libcudart.so")
        raw = C.c_void_p()
        if cudart.cudaMalloc(C.byref(raw), C.c_size_t(self.total_bytes)) != 0:
            raise RuntimeError("cudaMalloc failed")
        self._ipc_raw = raw.value
        handle = (C.c_char * 64)()
        native.check(lib.conef_ipc_get_handle(raw.value, C.cast(handle, C.c_void_p)), "ipc_get_handle")
        gathered: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle.raw), group=self.group)
        ptrs = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                ptrs.append(raw.value)
                continue
            out = C.c_void_p()
            hb = (C.c_char * 64).from_buffer_copy(h)
            native.check(lib.conef_ipc_open_handle(C.cast(hb, C.c_void_p), C.byref(out)), "ipc_open_handle")
            ptrs.append(out.value)
            self._ipc_ptrs.append(out.value)
        self.base_ptrs = ptrs
        self.local_bytes = _tensor_from_ptr(raw.value, self.total_bytes, self.device)

    # -- views and pointer tables ----------------------------------------------
    def _build_pointer_tables(self):
        rows = [[p for p in self.base_ptrs]]  # row 0: flag arrays
        for slot in range(2):
            for reg in range(len(self.region_floats)):
                rows.append([p + self.offsets[slot][reg] for p in self.base_ptrs])
        self.ptr_table = torch.tensor(rows, dtype=torch.int64, device=self.device)

    def flags_ptr(self) -> int:
        return self.base_ptrs[self.rank]

    def peer_flags_dev(self) -> int:
        return self.ptr_table[0].data_ptr()

    def peer_ptrs_dev(self, slot: int, region: int) -> int:
        return self.ptr_table[1 + slot * len(self.region_floats) + region].data_ptr()

    def local(self, slot: int, region: int) -> torch.Tensor:
        off = self.offsets[slot][region]
        nf = self.region_floats[region]
        return self.local_bytes[off : off + nf * 4].view(torch.float32)

    def close(self):
        if self.backend == "ipc":
            lib = native.lib()
            for p in self._ipc_ptrs:
                lib.conef_ipc_close_handle(p)
            self._ipc_ptrs = []


class LocalSlots:
    """The slot / region layout of :class:`SymmBuffer` in plain device memory for a group of one:
    the same kernels then run on one GPU with pointer tables of a single entry and no flags."""

    backend = "local"

    def __init__(self, region_floats: Sequence[int], device: torch.device):
        self.device, self.world, self.rank = device, 1, 0
        self.region_floats = list(region_floats)
        self.offsets: List[List[int]] = []
        cursor = 0
        for _slot in range(2):
            row = []
            for nf in self.region_floats:
                row.append(cursor)
                cursor = _round_up(cursor + nf * 4, ALIGN)
            self.offsets.append(row)
        self.total_bytes = cursor
        self.local_bytes = torch.zeros(max(cursor, ALIGN), dtype=torch.uint8, device=device)
        base = self.local_bytes.data_ptr()
        rows = [[base + self.offsets[slot][reg]] for slot in range(2) for reg in range(len(self.region_floats))]
        self.ptr_table = torch.tensor(rows, dtype=torch.int64, device=device)

    def peer_ptrs_dev(self, slot: int, region: int) -> int:
        return self.ptr_table[slot * len(self.region_floats) + region].data_ptr()

    def local(self, slot: int, region: int) -> torch.Tensor:
        off = self.offsets[slot][region]
        nf = self.region_floats[region]
        return self.local_bytes[off : off + nf * 4].view(torch.float32)


def _tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    """Wrap raw device memory as a uint8 tensor (no ownership)."""

    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {
        "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}
    return torch.as_tensor(h, device=device)


def comm_backend_choice() -> str:
    """``CONEF_COMM``: ``auto`` (default), ``symm``, ``ipc`` or ``nccl``."""
    return os.environ.get("CONEF_COMM", "auto")
