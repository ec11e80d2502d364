"""Small helpers shared by the example drivers: rank queries, result pickling, JSON-lines logging.

Counterparts of the reference's ``examples/BertPretraining/utils.py:20-65`` and
``examples/*/utils/pickle.py:12-51``.
"""
from __future__ import annotations

import json
import os
import pickle
import sys
import time

import torch.distributed as dist


def get_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def is_main_process() -> bool:
    return get_rank() == 0


def barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def mkdir_by_main_process(path: str) -> None:
    if is_main_process():
        os.makedirs(path, exist_ok=True)
    barrier()


def format_step(step) -> str:
    if isinstance(step, str):
        return step
    names = ("Training Epoch", "Training Iteration", "Validation Iteration")
    return " ".join(f"{n}: {v}" for n, v in zip(names, step))


def make_directory(path: str) -> None:
    os.makedirs(path, exist_ok=True)


def save_obj(obj, name: str) -> None:
    with open(name if name.endswith(".pkl") else name + ".pkl", "wb") as fh:
        pickle.dump(obj, fh, pickle.HIGHEST_PROTOCOL)


def load_obj(name: str):
    with open(name if name.endswith(".pkl") else name + ".pkl", "rb") as fh:
        return pickle.load(fh)


class JsonLogger:
    """One JSON object per line to a file and/or stdout; only rank 0 writes."""

    def __init__(self, path: str = None, stdout: bool = True):
        self.fh = open(path, "a") if (path and is_main_process()) else None
        self.stdout = stdout and is_main_process()
        self.t0 = time.time()

    def log(self, step, **data) -> None:
        rec = {"elapsed_s": round(time.time() - self.t0, 3), "step": step, **data}
        line = json.dumps(rec)
        if self.fh:
            self.fh.write(line + "\n")
            self.fh.flush()
        if self.stdout:
            sys.stdout.write(line + "\n")

    def close(self) -> None:
        if self.fh:
            self.fh.close()
