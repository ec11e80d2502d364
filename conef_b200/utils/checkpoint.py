"""Checkpoint / resume and graceful stop.

The reference's BERT driver saves ``ckpt_<step>.pt`` with model, optimizer, data position and
keeps the three most recent files (``run_pretraining_conef.py:717-739``), finds the newest one
to resume (``:419-438``), and turns SIGTERM into "checkpoint, then exit" (``:66-79``).  It never
saves the hook state; here the reducer's ``state_dict()`` (error buffers, sketches, P/Q memory,
shared RNG, iteration counter) is part of every checkpoint, so a resumed run continues with
the same compression state.
"""
from __future__ import annotations

import glob
import logging
import os
import re
import signal
from typing import Any, Dict, Optional

import torch


class GracefulStop:
    """Installs SIGTERM / SIGINT handlers that only set a flag the training loop polls."""

    def __init__(self, signals=(signal.SIGTERM,)):
        self.requested = False
        self._old = {}
        for sig in signals:
            try:
                self._old[sig] = signal.signal(sig, self._handler)
            except ValueError:          # not in the main thread
                pass

    def _handler(self, signum, frame):
        self.requested = True

    def restore(self):
        for sig, old in self._old.items():
            signal.signal(sig, old)


def checkpoint_path(directory: str, step: int) -> str:
    return os.path.join(directory, f"ckpt_{step}.pt")


def latest_checkpoint(directory: str) -> Optional[str]:
    best, best_step = None, -1
    for f in glob.glob(os.path.join(directory, "ckpt_*.pt")):
        m = re.search(r"ckpt_(\d+)\.pt$", f)
        if m and int(m.group(1)) > best_step:
            best, best_step = f, int(m.group(1))
    return best


def save_checkpoint(directory: str, step: int, *, model, optimizer=None, reducer_state=None, scheduler=None,
                    extra: Optional[Dict[str, Any]] = None, keep_last: int = 3, rank: int = 0) -> Optional[str]:
    """Rank 0 writes ``ckpt_<step>.pt`` atomically and prunes all but the newest ``keep_last``.

    With error feedback every rank has its own error memory: pass ``per_rank=True`` in
    ``extra`` to write ``ckpt_<step>.rank<r>.pt`` side files with each rank's reducer state
    (atomically, before rank 0 publishes the main file when a process group is up; they are pruned
    together with their step).  Without ``per_rank`` every rank resumes from rank 0's error memory.
    """
    extra = dict(extra or {})
    per_rank = bool(extra.pop("per_rank", False))
    os.makedirs(directory, exist_ok=True)
    module = getattr(model, "module", model)
    if per_rank and reducer_state is not None and rank != 0:
        side = os.path.join(directory, f"ckpt_{step}.rank{rank}.pt")
        torch.save({"reducer": reducer_state.state_dict()}, side + ".tmp")
        os.replace(side + ".tmp", side)
    if per_rank:
        # the main file is the marker of a complete checkpoint: publish it after every side file
        try:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                dist.barrier()
        except Exception:  # noqa: BLE001 - a checkpoint must not fail because of the barrier
            pass
    if rank != 0:
        return None
    blob = {"model": module.state_dict(), "step": step, "extra": extra,
            "optimizer": optimizer.state_dict() if optimizer is not None else None,
            "scheduler": scheduler.state_dict() if scheduler is not None and hasattr(scheduler, "state_dict") else None,
            "reducer": reducer_state.state_dict() if reducer_state is not None else None}
    path = checkpoint_path(directory, step)
    tmp = path + ".tmp"
    torch.save(blob, tmp)
    os.replace(tmp, path)
    files = sorted(glob.glob(os.path.join(directory, "ckpt_*.pt")),
                   key=lambda f: int(re.search(r"ckpt_(\d+)", f).group(1)))
    files = [f for f in files if ".rank" not in f]
    for old in files[:-keep_last] if keep_last > 0 else []:
        os.remove(old)
        for side in glob.glob(old[: -len(".pt")] + ".rank*.pt"):     # the step's per-rank side files
            os.remove(side)
    return path


def load_checkpoint(path: str, *, model, optimizer=None, reducer_state=None, scheduler=None, device=None,
                    rank: int = 0) -> Dict[str, Any]:
    blob = torch.load(path, map_location="cpu", weights_only=False)
    getattr(model, "module", model).load_state_dict(blob["model"])
    if optimizer is not None and blob.get("optimizer") is not None:
        optimizer.load_state_dict(blob["optimizer"])
    if scheduler is not None and blob.get("scheduler") is not None:
        scheduler.load_state_dict(blob["scheduler"])
    if reducer_state is not None:
        side = path.replace(".pt", f".rank{rank}.pt")
        red = blob.get("reducer")
        if rank != 0 and os.path.exists(side):
            red = torch.load(side, map_location="cpu", weights_only=False)["reducer"]
        elif rank != 0 and red is not None:
            logging.getLogger(__name__).warning(
                "rank %d: %s not found, resuming the reducer from rank 0's error memory", rank, os.path.basename(side))
        if red is not None:
            reducer_state.load_state_dict(red, device=device)
    return {"step": blob.get("step", 0), "extra": blob.get("extra", {})}
