"""Phase timers and NVTX ranges for the hooks and training loops.

The reference only takes wall-clock time per epoch (``examples/ImageClassification/main.py:297-299``).
Here a :class:`PhaseTimer` brackets named phases with CUDA events on the stream that runs
them (no host synchronisation until ``summary()`` is asked for), and ``exposed_comm_ms``
derives the communication time a step cannot hide: step time with the reducer minus step time
with a no-op reducer, max over ranks.
"""
from __future__ import annotations

import contextlib
import time
from collections import defaultdict
from typing import Dict, List, Tuple

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when CUDA is available, otherwise a no-op."""
    use = torch.cuda.is_available()
    if use:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if use:
            torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """Accumulates device time per named phase with CUDA events (wall clock on CPU)."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self._events: Dict[str, List[Tuple["torch.cuda.Event", "torch.cuda.Event"]]] = defaultdict(list)
        self._host: Dict[str, float] = defaultdict(float)
        self._counts: Dict[str, int] = defaultdict(int)

    @contextlib.contextmanager
    def phase(self, name: str, device=None):
        if not self.enabled:
            yield
            return
        self._counts[name] += 1
        if torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda"):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            with nvtx_range(name):
                yield
            end.record()
            self._events[name].append((start, end))
        else:
            t0 = time.perf_counter()
            yield
            self._host[name] += (time.perf_counter() - t0) * 1e3

    def summary(self) -> Dict[str, Dict[str, float]]:
        """{phase: {"ms": total, "calls": n, "ms_per_call": mean}}; synchronises the device once."""
        if self._events:
            torch.cuda.synchronize()
        out = {}
        for name in set(self._events) | set(self._host):
            ms = self._host.get(name, 0.0) + sum(s.elapsed_time(e) for s, e in self._events.get(name, []))
            n = max(1, self._counts[name])
            out[name] = {"ms": ms, "calls": self._counts[name], "ms_per_call": ms / n}
        return out

    def reset(self) -> None:
        self._events.clear()
        self._host.clear()
        self._counts.clear()


def max_over_ranks(value: float, device=None) -> float:
    """Max of a host scalar over all ranks (identity without a process group)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def exposed_comm_ms(step_ms_with_reducer: float, step_ms_noop_reducer: float) -> float:
    """Communication (and compression) time that backward could not hide, per step."""
    return max(0.0, step_ms_with_reducer - step_ms_noop_reducer)
