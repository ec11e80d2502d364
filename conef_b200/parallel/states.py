"""Hook state objects: hyper-parameters plus the persistent per-bucket buffers.

Field names and layouts follow the reference so that checkpoints keep the
same structure:

  PowerSGDState            communication/powerSGD_hook.py:89-277
  hPowerSGDState           communication/hPowerSGD_hook.py:101-271
  RandomBlockState         communication/RandomBlock_hook.py:16-135
  UnbiasedRandomBlockState communication/UnbiasedRandomBlock_hook.py:12-95
  unbiasedMtrxState        communication/unbiasedMtrx_hook.py:47-139

``error_dict[bucket]`` is a 1-D bucket-length tensor (classic EF), a dict
``{cnt: compressor}`` (PowerSGD family with a compressed error store) or a
list of tensors / compressors (random block).  ``p_memory_dict`` /
``q_memory_dict`` hold flat 1-D tensors.  ``rng`` is a NumPy ``RandomState``
that every rank advances identically.

Additions over the reference: ``error_compressor`` selects the compressed
error store; ``state_dict()`` / ``load_state_dict()`` exist on the states
themselves; pickling drops ``process_group`` and all device-side caches.
"""
from __future__ import annotations

import logging
from typing import Any, Dict

import numpy as np
import torch

from ..compressors.other import ERROR_COMPRESSORS

logger = logging.getLogger(__name__)

# slots that never go into a checkpoint / pickle
_RUNTIME_SLOTS = ("process_group", "_engines", "_timers", "_wire", "_status_probe", "_process_iters", "_sig_seen")


def _to_cpu(obj):
    if torch.is_tensor(obj):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_to_cpu(v) for v in obj]
    if hasattr(obj, "state_dict") and not isinstance(obj, np.random.RandomState):
        return {"__compressor__": type(obj).__name__, "state": obj.state_dict()}
    return obj


def _restore(saved, live, device):
    """Rebuild ``saved`` (output of _to_cpu) on ``device``; reuse ``live`` objects when shapes match."""
    from .. import compressors as C

    if torch.is_tensor(saved):
        if torch.is_tensor(live) and live.shape == saved.shape:
            live.copy_(saved)
            return live
        return saved.to(device)
    if isinstance(saved, dict) and "__compressor__" in saved:
        cls = getattr(C, saved["__compressor__"])
        obj = live if isinstance(live, cls) else cls.__new__(cls)
        obj.load_state_dict(saved["state"])
        if hasattr(obj, "to") and not isinstance(live, cls):
            obj.to(device)
        return obj
    if isinstance(saved, dict):
        live = live if isinstance(live, dict) else {}
        return {k: _restore(v, live.get(k), device) for k, v in saved.items()}
    if isinstance(saved, list):
        live = live if isinstance(live, list) else []
        return [_restore(v, live[i] if i < len(live) else None, device) for i, v in enumerate(saved)]
    return saved


class _StateBase:
    __slots__ = ()

    def _init_runtime(self):
        self._engines = {}
        self._timers = None              # utils.tracing.PhaseTimer when phase timing is on
        self._wire = [0, 0, 0]           # fp32 elements sent, elements before compression, compressed steps
        self._status_probe = None        # (pinned host copy of the device status word, its event)
        self._process_iters = 0      # reduced iterations seen by this process (not persisted)
        self._sig_seen = set()       # buckets whose layout was checked in this process
        self.bucket_signatures = {}  # persisted: bucket index -> (numel, parameter shapes)

    def in_warmup(self, start_iter: int, bucket=None) -> bool:
        """Plain all-reduce while ``iter < start_iter`` - and, after a resume, for as long as a
        bucket does not have the layout its saved state was built for: DDP rebuilds its buckets
        after the first iteration of a process, so per-bucket state restored from a checkpoint
        only lines up with the rebuilt layout."""
        if self.iter < start_iter:
            return True
        if bucket is None:
            return False
        bidx = bucket.index()
        if bidx in self._sig_seen:
            return False
        sig = (bucket.buffer().numel(), tuple(tuple(g.shape) for g in bucket.gradients()))
        known = self.bucket_signatures.get(bidx)
        if known is not None and known != sig and self._process_iters < 1:
            return True              # pre-rebuild layout of a resumed run: leave the saved state alone
        self.bucket_signatures[bidx] = sig
        self._sig_seen.add(bidx)
        return False

    # iteration counter: advances once per step, on the last bucket
    def maybe_increase_iter(self, bucket) -> None:
        if bucket.is_last():
            self.iter += 1
            self._process_iters += 1
        start = getattr(self, "start_powerSGD_iter", None)
        if start is None:
            start = getattr(self, "start_compression_iter")
        if self.iter == start and bucket.is_last():
            logger.info("Start to apply the compressed hook after %d iterations.", self.iter)

    # -- pickling / checkpointing ------------------------------------------
    def _persisted_slots(self):
        names = []
        for klass in type(self).__mro__:
            names.extend(getattr(klass, "__slots__", ()))
        return [n for n in dict.fromkeys(names) if n not in _RUNTIME_SLOTS]

    def __getstate__(self) -> Dict[str, Any]:
        return {n: getattr(self, n) for n in self._persisted_slots() if hasattr(self, n)}

    def __setstate__(self, d: Dict[str, Any]) -> None:
        self.process_group = None
        self._init_runtime()
        for k, v in d.items():
            setattr(self, k, v)

    def state_dict(self) -> Dict[str, Any]:
        """CPU copy of everything needed to resume: hyper-parameters, iteration
        counter, RNG state, error buffers, P/Q memory."""
        out = {}
        for n in self._persisted_slots():
            v = getattr(self, n)
            if isinstance(v, np.random.RandomState):
                out[n] = v.get_state()
            else:
                out[n] = _to_cpu(v)
        return out

    def load_state_dict(self, d: Dict[str, Any], device=None) -> None:
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
        for n, v in d.items():
            if n == "rng":
                self.rng.set_state(v)
            elif n in ("error_dict", "p_memory_dict", "q_memory_dict", "compressed_tensor_memory"):
                setattr(self, n, _restore(v, getattr(self, n, None), device))
            else:
                setattr(self, n, v)
        # device tables are rebuilt against the restored tensors on the next call
        self._engines = {}
        self._sig_seen = set()
        self._process_iters = 0

    # -- metrics -----------------------------------------------------------
    def account_wire(self, numel_sent: int, numel_before: int, bucket) -> None:
        """Called by every compressed hook invocation: what this bucket puts on the wire."""
        self._wire[0] += int(numel_sent)
        self._wire[1] += int(numel_before)
        if bucket.is_last():
            self._wire[2] += 1

    def wire_bytes_per_step(self) -> float:
        """Bytes (fp32 payloads) this rank contributes to the collectives of one compressed step,
        averaged over the compressed steps of this process; 0 before the first one."""
        return 4.0 * self._wire[0] / self._wire[2] if self._wire[2] else 0.0

    def wire_compression_rate(self) -> float:
        """Gradient elements per element sent, over the compressed steps of this process."""
        return self._wire[1] / self._wire[0] if self._wire[0] else 0.0

    def enable_phase_timing(self, enabled: bool = True) -> None:
        """Time the phases of every compressed hook call with CUDA events on the hook's stream
        (P pass, reduction + Gram-Schmidt + Q pass, reduction + decompress).  While it is on, the
        native executor issues the phases as separate calls instead of replaying its graph."""
        from ..utils.tracing import PhaseTimer
        self._timers = PhaseTimer() if enabled else None

    def phase_summary(self) -> Dict[str, Dict[str, float]]:
        """``{phase: {"ms", "calls", "ms_per_call"}}`` since phase timing was switched on."""
        return self._timers.summary() if self._timers is not None else {}

    def ef_buffer_bytes(self) -> int:
        """Bytes of persistent error-feedback state (the ConEF headline metric)."""
        def size(o):
            if torch.is_tensor(o):
                return o.numel() * o.element_size()
            if isinstance(o, dict):
                return sum(size(v) for v in o.values())
            if isinstance(o, list):
                return sum(size(v) for v in o)
            if hasattr(o, "nbytes"):
                return int(o.nbytes())
            return 0
        return size(getattr(self, "error_dict", {}))

    def check_status(self) -> None:
        """Raise if a device-side bounded wait gave up (peer never signalled).  Synchronises."""
        self._status_probe = None
        for eng in self._engines.values():
            eng.check_status()

    # The hook path checks for itself, without a host synchronisation: the last bucket of a step
    # enqueues a copy of the device status word into pinned memory behind its kernels, and every
    # later hook call looks at that copy once its event has completed.
    def post_status(self, status_dev, stream) -> None:
        probe = self._status_probe
        if probe is None:
            host = torch.zeros(status_dev.numel(), dtype=status_dev.dtype).pin_memory()
            probe = self._status_probe = [host, None, status_dev]
        elif probe[1] is not None:
            if not probe[1].query():
                return                   # the previous copy has not landed yet: keep waiting for it
            self.poll_status()
        with torch.cuda.stream(stream):
            probe[0].copy_(status_dev, non_blocking=True)
            probe[1] = torch.cuda.Event()
            probe[1].record(stream)
        probe[2] = status_dev

    def poll_status(self) -> None:
        """Raise if the status word copied at the end of an earlier step shows a wait that gave up."""
        probe = self._status_probe
        if probe is None or probe[1] is None or not probe[1].query():
            return
        probe[1] = None
        code = int(probe[0][0])
        if code != 0:
            probe[2].zero_()
            raise RuntimeError(
                f"device-side wait gave up (status {code}) in an earlier step: a peer rank did not signal in "
                "time; the gradients of that step are not valid")


def _check_error_compressor(kind):
    if kind not in ERROR_COMPRESSORS:
        raise ValueError(f"unknown error_compressor {kind!r}; choose from {ERROR_COMPRESSORS}")


class PowerSGDState(_StateBase):
    __slots__ = [
        "process_group", "matrix_approximation_rank", "start_powerSGD_iter", "min_compression_rate",
        "orthogonalization_epsilon", "use_error_compression", "beta", "sketch_size",
        "use_error_feedback", "warm_start", "rng", "error_dict", "p_memory_dict", "q_memory_dict",
        "iter", "total_numel_before_compression", "total_numel_after_compression",
        "compression_stats_logging_frequency", "next_stats_report",
        # additions
        "error_compressor", "error_rank", "hash_seed", "_engines", "_timers", "_wire", "_status_probe", "_process_iters", "_sig_seen",
        "bucket_signatures",
    ]

    def __init__(self, process_group, matrix_approximation_rank=1, start_powerSGD_iter=1_000,
                 min_compression_rate=2, use_error_compression=False, beta=0.9, sketch_size=0.5,
                 use_error_feedback=True, warm_start=True, orthogonalization_epsilon=0, random_seed=0,
                 compression_stats_logging_frequency=10_000, error_compressor="count_sketch",
                 error_rank=None, hash_seed=0):
        logger.info(
            "PowerSGD config: matrix_approximation_rank = %s; start_powerSGD_iter = %s; "
            "min_compression_rate = %s; orthogonalization_epsilon = %s; use_error_feedback = %s; "
            "use_error_compression = %s (%s, size %s, beta %s); warm_start = %s; random_seed = %s",
            matrix_approximation_rank, start_powerSGD_iter, min_compression_rate, orthogonalization_epsilon,
            use_error_feedback, use_error_compression, error_compressor, sketch_size, beta, warm_start,
            random_seed)
        self.process_group = process_group
        self.matrix_approximation_rank = matrix_approximation_rank
        # DDP rebuilds its buckets after the first iteration, which would
        # invalidate per-bucket error / P / Q memory created at iteration 1.
        if (use_error_feedback or warm_start) and start_powerSGD_iter <= 1:
            raise ValueError(
                "Expect `start_powerSGD_iter` > 1 if `use_error_feedback` or `warm_start` is enabled, "
                "because PowerSGD can only be applied after the first two iterations in DDP.")
        if use_error_compression and not use_error_feedback:
            raise ValueError("`use_error_compression` requires `use_error_feedback`.")
        _check_error_compressor(error_compressor)
        self.start_powerSGD_iter = start_powerSGD_iter
        self.min_compression_rate = min_compression_rate
        self.use_error_feedback = use_error_feedback
        self.use_error_compression = use_error_compression
        self.beta = beta
        self.sketch_size = sketch_size
        self.warm_start = warm_start
        self.orthogonalization_epsilon = orthogonalization_epsilon
        self.rng = np.random.RandomState(random_seed)
        self.error_dict = {}
        self.p_memory_dict = {}
        self.q_memory_dict = {}
        self.iter = 0
        self.total_numel_before_compression = 0
        self.total_numel_after_compression = 0
        self.compression_stats_logging_frequency = max(1, compression_stats_logging_frequency)
        self.next_stats_report = 0
        self.error_compressor = error_compressor
        self.error_rank = error_rank if error_rank is not None else matrix_approximation_rank
        self.hash_seed = hash_seed
        self._init_runtime()

    def compression_stats(self):
        """(compression rate, numel before, numel after), as the reference's ``compression_stats``."""
        rate = (self.total_numel_before_compression / self.total_numel_after_compression
                if self.total_numel_after_compression > 0 else 0)
        return rate, self.total_numel_before_compression, self.total_numel_after_compression

    def clean_error(self, alpha: float = 0.0) -> None:
        """Scale every remembered error by ``alpha`` (0 forgets it).  Works for
        both layouts; the reference's version only handles the sketch layout."""
        for entry in self.error_dict.values():
            if torch.is_tensor(entry):
                entry.mul_(alpha)
            else:
                for comp in (entry.values() if isinstance(entry, dict) else entry):
                    comp.mul_(alpha) if torch.is_tensor(comp) else comp.clean(alpha)


class hPowerSGDState(PowerSGDState):
    """PowerSGD whose per-matrix error memory is sparsified by top-k after every
    step (``topk_ratio``), or — an addition — kept as low-rank factors."""

    __slots__ = ["topk_ratio"]

    def __init__(self, process_group, matrix_approximation_rank=1, start_powerSGD_iter=1_000,
                 min_compression_rate=2, use_error_compression=False, use_error_feedback=True,
                 topk_ratio=0.4, warm_start=True, orthogonalization_epsilon=0, random_seed=0,
                 compression_stats_logging_frequency=10_000, error_compressor="topk", error_rank=None):
        super().__init__(process_group, matrix_approximation_rank, start_powerSGD_iter, min_compression_rate,
                         use_error_compression=use_error_compression, beta=0.0, sketch_size=0.0,
                         use_error_feedback=use_error_feedback, warm_start=warm_start,
                         orthogonalization_epsilon=orthogonalization_epsilon, random_seed=random_seed,
                         compression_stats_logging_frequency=compression_stats_logging_frequency,
                         error_compressor=error_compressor, error_rank=error_rank)
        self.topk_ratio = topk_ratio


class RandomBlockState(_StateBase):
    __slots__ = [
        "process_group", "compression_ratio", "start_compression_iter", "n_blocks",
        "use_error_compression", "beta", "sketch_size", "use_error_feedback", "rng", "error_dict",
        "iter", "compression_stats_logging_frequency", "next_stats_report", "compressed_tensor_memory",
        "error_compressor", "hash_seed", "_engines", "_timers", "_wire", "_status_probe", "_process_iters", "_sig_seen",
        "bucket_signatures",
    ]

    def __init__(self, process_group, compression_ratio=0.1, start_compression_iter=1_000,
                 use_error_compression=False, beta=0.9, sketch_size=0.5, use_error_feedback=True,
                 random_seed=42, compression_stats_logging_frequency=10_000,
                 error_compressor="count_sketch", hash_seed=0):
        logger.info(
            "RandomBlock config: compression_ratio = %s; start_compression_iter = %s; "
            "use_error_feedback = %s; use_error_compression = %s (%s, size %s, beta %s)",
            compression_ratio, start_compression_iter, use_error_feedback, use_error_compression,
            error_compressor, sketch_size, beta)
        if start_compression_iter <= 1:
            raise ValueError(
                "Expect `start_compression_iter` > 1, because compression can only be applied after "
                "the first two iterations in DDP.")
        if use_error_compression and not use_error_feedback:
            raise ValueError("Expect `use_error_feedback` = True when `use_error_compression` is True.")
        _check_error_compressor(error_compressor)
        self.process_group = process_group
        self.compression_ratio = compression_ratio
        self.start_compression_iter = start_compression_iter
        self.n_blocks = None
        self.use_error_feedback = use_error_feedback
        self.use_error_compression = use_error_compression
        self.beta = beta
        self.sketch_size = sketch_size
        self.rng = np.random.RandomState(random_seed)
        self.error_dict = {}
        self.iter = 0
        self.compression_stats_logging_frequency = max(1, compression_stats_logging_frequency)
        self.next_stats_report = 0
        self.compressed_tensor_memory = {}
        self.error_compressor = error_compressor
        self.hash_seed = hash_seed
        self._init_runtime()

    def clean_error(self, alpha: float = 0.0) -> None:
        for entry in self.error_dict.values():
            for comp in entry:
                comp.mul_(alpha) if torch.is_tensor(comp) else comp.clean(alpha)


class UnbiasedRandomBlockState(_StateBase):
    __slots__ = [
        "process_group", "compression_ratio", "start_compression_iter", "rng", "iter",
        "compression_stats_logging_frequency", "next_stats_report", "compressed_tensor_memory",
        "_engines", "_timers", "_wire", "_status_probe", "_process_iters", "_sig_seen",
        "bucket_signatures",
    ]

    def __init__(self, process_group, compression_ratio=0.1, start_compression_iter=1_000, random_seed=42,
                 compression_stats_logging_frequency=10_000):
        if start_compression_iter <= 1:
            raise ValueError(
                "Expect `start_compression_iter` > 1, because compression can only be applied after "
                "the first two iterations in DDP.")
        self.process_group = process_group
        self.compression_ratio = compression_ratio
        self.start_compression_iter = start_compression_iter
        self.rng = np.random.RandomState(random_seed)
        self.iter = 0
        self.compression_stats_logging_frequency = max(1, compression_stats_logging_frequency)
        self.next_stats_report = 0
        self.compressed_tensor_memory = {}
        self._init_runtime()


class unbiasedMtrxState(_StateBase):
    __slots__ = [
        "process_group", "matrix_approximation_rank", "start_powerSGD_iter", "min_compression_rate",
        "orthogonalization_epsilon", "rng", "p_memory_dict", "q_memory_dict", "iter",
        "total_numel_before_compression", "total_numel_after_compression",
        "compression_stats_logging_frequency", "next_stats_report",
        "_engines", "_timers", "_wire", "_status_probe", "_process_iters", "_sig_seen",
        "bucket_signatures",
    ]

    def __init__(self, process_group, matrix_approximation_rank=1, start_powerSGD_iter=1_000,
                 min_compression_rate=2, random_seed=421, compression_stats_logging_frequency=10_000):
        if start_powerSGD_iter <= 1:
            raise ValueError("Expect `start_powerSGD_iter` > 1: DDP rebuilds its buckets after iteration 1.")
        self.process_group = process_group
        self.matrix_approximation_rank = matrix_approximation_rank
        self.start_powerSGD_iter = start_powerSGD_iter
        self.min_compression_rate = min_compression_rate
        self.orthogonalization_epsilon = 0
        self.rng = np.random.RandomState(random_seed)
        self.p_memory_dict = {}
        self.q_memory_dict = {}
        self.iter = 0
        self.total_numel_before_compression = 0
        self.total_numel_after_compression = 0
        self.compression_stats_logging_frequency = max(1, compression_stats_logging_frequency)
        self.next_stats_report = 0
        self._init_runtime()

    def compression_stats(self):
        rate = (self.total_numel_before_compression / self.total_numel_after_compression
                if self.total_numel_after_compression > 0 else 0)
        return rate, self.total_numel_before_compression, self.total_numel_after_compression
