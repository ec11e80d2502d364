"""Reducer registry: ``--grad_reducer`` name -> State + hook, registered on a DDP model.

Same eight names and argument fields as the reference's
``examples/*/get_comm_hooks.py:9-126`` (``allreduce``, ``ef_randomblock``,
``conef_randomblock``, ``unbiased_randomblock``, ``ef_powersgd``,
``hefsgd_powersgd``, ``conef_powersgd``, ``unbiased_mtrx``), plus
``batched_powersgd`` and ``c2cs_powersgd`` for the two extra hooks of
``communication/powerSGD_hook.py``, and an optional ``args.error_compressor``
(``count_sketch`` / ``count_sketch3`` / ``half_count_sketch`` / ``topk`` /
``quant8`` / ``lowrank``) selecting what the error buffer is stored as.
"""
from __future__ import annotations

from . import hooks
from .states import (PowerSGDState, RandomBlockState, UnbiasedRandomBlockState, hPowerSGDState,
                     unbiasedMtrxState)

REDUCERS = ("allreduce", "ef_randomblock", "conef_randomblock", "unbiased_randomblock", "ef_powersgd",
            "hefsgd_powersgd", "conef_powersgd", "unbiased_mtrx", "batched_powersgd", "c2cs_powersgd")


def _get(args, name, default):
    return getattr(args, name, default)


def build_state_and_hook(args):
    """Return ``(state, hook)`` for ``args.grad_reducer`` (``(None, None)`` for plain all-reduce)."""
    name = args.grad_reducer.lower()
    start = args.start_compression_iter
    err = _get(args, "error_compressor", None)
    if name == "allreduce":
        return None, None
    if name == "ef_randomblock":
        return RandomBlockState(None, compression_ratio=args.compression_ratio,
                                start_compression_iter=start), hooks.RandomBlock_hook
    if name == "conef_randomblock":
        return RandomBlockState(None, compression_ratio=args.compression_ratio, start_compression_iter=start,
                                use_error_compression=True, sketch_size=args.sketch_size, beta=args.beta,
                                error_compressor=err or "count_sketch"), hooks.RandomBlock_hook
    if name == "unbiased_randomblock":
        return UnbiasedRandomBlockState(None, compression_ratio=args.compression_ratio,
                                        start_compression_iter=start), hooks.UnbiasedRandomBlock_hook
    common = dict(matrix_approximation_rank=_get(args, "matrix_approximation_rank", 1),
                  start_powerSGD_iter=start, min_compression_rate=_get(args, "min_compression_rate", 2))
    eps = _get(args, "orthogonalization_epsilon", 0)
    if name == "ef_powersgd":
        return PowerSGDState(None, orthogonalization_epsilon=eps, **common), hooks.powerSGD_hook
    if name == "batched_powersgd":
        return PowerSGDState(None, orthogonalization_epsilon=eps, **common), hooks.batched_powerSGD_hook
    if name == "hefsgd_powersgd":
        return hPowerSGDState(None, orthogonalization_epsilon=eps, use_error_compression=True,
                              topk_ratio=_get(args, "topk_ratio", 0.4), error_compressor=err or "topk",
                              error_rank=_get(args, "error_rank", None), **common), hooks.hpowerSGD_hook
    if name in ("conef_powersgd", "c2cs_powersgd"):
        state = PowerSGDState(None, orthogonalization_epsilon=eps, sketch_size=args.sketch_size, beta=args.beta,
                              use_error_compression=True, error_compressor=err or "count_sketch",
                              hash_seed=_get(args, "hash_seed", 0), **common)
        return state, (hooks.powerSGD_hook if name == "conef_powersgd" else hooks.C2CS_hook_v2)
    if name == "unbiased_mtrx":
        return unbiasedMtrxState(None, **common), hooks.UnbiasedMtrx_hook
    raise ValueError(f"Communication hook {args.grad_reducer!r} is not supported; choose from {REDUCERS}")


def get_comm_hooks(args, net, gpu=None):
    """Register the hook selected by ``args.grad_reducer`` on the DDP model ``net``.

    Returns the state (``None`` for plain all-reduce) so that the caller can
    checkpoint it or read its metrics."""
    state, hook = build_state_and_hook(args)
    if state is not None:
        net.register_comm_hook(state, hook)
    return state
