"""Tracing, checkpointing and small helpers."""
from .checkpoint import GracefulStop, latest_checkpoint, load_checkpoint, save_checkpoint
from .misc import (JsonLogger, barrier, get_rank, get_world_size, is_main_process, load_obj, make_directory,
                   mkdir_by_main_process, save_obj)
from .tracing import PhaseTimer, exposed_comm_ms, max_over_ranks, nvtx_range

__all__ = ["GracefulStop", "latest_checkpoint", "load_checkpoint", "save_checkpoint", "JsonLogger", "barrier",
           "get_rank", "get_world_size", "is_main_process", "load_obj", "make_directory", "mkdir_by_main_process",
           "save_obj", "PhaseTimer", "exposed_comm_ms", "max_over_ranks", "nvtx_range"]
