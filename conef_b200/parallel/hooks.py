"""DDP communication hooks: ``hook(state, bucket) -> Future``.

Register with ``ddp_model.register_comm_hook(state, hook)``.  Each hook runs a
plain averaged all-reduce until ``state.iter`` reaches the state's start
iteration, then compresses every bucket.

Two execution paths share the same semantics:

* **native** (CUDA buckets): a per-bucket plan drives a handful of grouped
  sm_100a kernels on a dedicated communication stream; the all-reduces of P, Q
  and of the staged uncompressed / random-block values are done by our own
  kernels over NVLink peer memory when symmetric memory is available (NCCL
  otherwise).  See :mod:`conef_b200.parallel.engine`.
* **torch** (CPU buckets over gloo, or ``CONEF_BACKEND=torch``): PyTorch ops and
  ``dist.all_reduce`` in the reference's op order; this is the numerics oracle
  and the baseline arm of the benchmarks.

Behavioural spec (reference project paths):
  powerSGD_hook / batched_powerSGD_hook / C2CS_hook_v2   communication/powerSGD_hook.py:280,583,791
  hpowerSGD_hook                                         communication/hPowerSGD_hook.py:274
  RandomBlock_hook                                       communication/RandomBlock_hook.py:138
  UnbiasedRandomBlock_hook                               communication/UnbiasedRandomBlock_hook.py:98
  UnbiasedMtrx_hook                                      communication/unbiasedMtrx_hook.py:143

torch >= 2 bucket API: ``bucket.buffer()``, ``.index()``, ``.gradients()``,
``.is_last()``; the returned future resolves to the bucket tensor itself.
"""

import logging
import math
from typing import List

import torch
import torch.distributed as dist

from ..compressors import DenseCS, make_error_compressor
from ..ops import native
from ..ops import reference as ref
from . import plan as planlib
from .states import (PowerSGDState, RandomBlockState, UnbiasedRandomBlockState, hPowerSGDState,
                     unbiasedMtrxState)

logger = logging.getLogger(__name__)

# Baseline switch: block the host after every bucket on the PyTorch-ops path, as the
# reference does (communication/powerSGD_hook.py:552-553).  Off in the product path.
SYNC_EVERY_BUCKET = False


# Measurement switch: with BYPASS set every hook returns the bucket as it is (no compression,
# no communication), so that "step time - step time with BYPASS" is the time the hook leaves
# exposed on the critical path of a training step.  Gradients are then not synchronised.
BYPASS = False


def _measurable(hook):
    import functools

    @functools.wraps(hook)
    def wrapped(state, bucket):
        if BYPASS:
            state.maybe_increase_iter(bucket)
            return _done(bucket.buffer())
        return hook(state, bucket)
    return wrapped


# --------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------
def _group(state):
    return state.process_group if state.process_group is not None else dist.group.WORLD


def _done(tensor: torch.Tensor) -> torch.futures.Future[torch.Tensor]:
    """Future already holding ``tensor``; for CUDA tensors it carries an event on
    the current stream, so consumers order themselves after the queued work."""
    if tensor.is_cuda:
        if SYNC_EVERY_BUCKET:
            torch.cuda.synchronize(tensor.device)
        fut = torch.futures.Future(devices=[tensor.device])
    else:
        fut = torch.futures.Future()
    fut.set_result(tensor)
    return fut


def allreduce_fut(group, tensor: torch.Tensor) -> torch.futures.Future[torch.Tensor]:
    """Averaged all-reduce of ``tensor`` (the warm-up path of every hook)."""
    ws = group.size()
    if ws == 1:
        return _done(tensor)
    tensor.div_(ws)
    return dist.all_reduce(tensor, group=group, async_op=True).get_future().then(lambda f: f.value()[0])


def _allreduce_sum(t: torch.Tensor, group) -> None:
    if group.size() > 1 and t.numel() > 0:
        dist.all_reduce(t, group=group)


def _report_compression_stats(bucket, state) -> None:
    if bucket.is_last() and state.iter >= state.next_stats_report:
        rate, before, after = state.compression_stats()
        logger.info("Compression stats: iter %d, total before compression %d, total after compression %d, "
                    "rate %s", state.iter, before, after, rate)
        state.next_stats_report = state.iter + state.compression_stats_logging_frequency


def _comm_stream(state, device) -> "torch.cuda.Stream":
    from .engine import comm_stream_for
    return comm_stream_for(device)


def _random_q_cpu(state, qs: List[torch.Tensor]) -> None:
    """Same-on-every-rank random Q: seed a forked CPU generator from the shared
    ``state.rng`` and copy to the device (communication/powerSGD_hook.py:475-494)."""
    with torch.random.fork_rng(devices=[]):
        torch.manual_seed(int(state.rng.randint(1_000_000_000)))
        for q in qs:
            q.copy_(torch.randn(*q.shape, device="cpu", dtype=q.dtype))


# --------------------------------------------------------------------------
# PowerSGD family, torch path
# --------------------------------------------------------------------------
def _make_matrix_compressor(state, n, m, device, transposed=False):
    kind = state.error_compressor
    N, D = (m, n) if transposed else (n, m)
    return make_error_compressor(
        kind, N, D, sketch_size=state.sketch_size, seed=getattr(state, "hash_seed", 0),
        topk_ratio=getattr(state, "topk_ratio", 0.4), rank=getattr(state, "error_rank", 4) or 4, device=device)


def _ef_coeffs(state):
    """(alpha for query, beta for update).  hPowerSGD feeds the whole remembered
    error back each step (alpha 1, beta 0); ConEF feeds back (1 - beta)."""
    if isinstance(state, hPowerSGDState):
        return 1.0, 0.0
    return 1.0 - state.beta, state.beta


def _powersgd_torch(state, bucket, group, *, transposed_sketch=False) -> torch.futures.Future[torch.Tensor]:
    ws = group.size()
    buf = bucket.buffer()
    device, dtype = buf.device, buf.dtype
    bidx = bucket.index()
    grads = bucket.gradients()
    plan = planlib.build_powersgd_plan(buf, grads, state.matrix_approximation_rank, state.min_compression_rate)
    state.total_numel_before_compression += plan.numel_before
    state.total_numel_after_compression += plan.numel_after
    state.account_wire(plan.numel_after, plan.numel_before, bucket)

    dense_ef = state.use_error_feedback and not state.use_error_compression
    conef = state.use_error_feedback and state.use_error_compression
    alpha, beta = _ef_coeffs(state)

    buf_copy = None
    if dense_ef:
        if bidx in state.error_dict and state.error_dict[bidx].numel() == buf.numel():
            buf.add_(state.error_dict[bidx])
        else:
            logger.info("A zero tensor of length %d that represents local error is created.", buf.numel())
            state.error_dict[bidx] = torch.zeros(buf.numel(), device=device, dtype=dtype)
        buf_copy = buf.clone()

    mats = [buf[e.g_off : e.g_off + e.numel].view(e.n, e.m) for e in plan.mats]
    copies = []
    if conef:
        comps = state.error_dict.setdefault(bidx, {})
        for cnt, (e, mat) in enumerate(zip(plan.mats, mats)):
            want = (e.m, e.n) if transposed_sketch else (e.n, e.m)
            if cnt not in comps or (comps[cnt].N, comps[cnt].D) != want:
                comps[cnt] = _make_matrix_compressor(state, e.n, e.m, device, transposed_sketch)
            comps[cnt].query(mat, alpha)
            copies.append(mat.clone())

    unc = (torch.cat([buf[s.g_off : s.g_off + s.numel] for s in plan.segs])
           if plan.segs else torch.empty(0, device=device, dtype=dtype))

    fresh = (not state.warm_start) or bidx not in state.p_memory_dict \
        or state.p_memory_dict[bidx].numel() != plan.total_p
    if fresh:
        if state.warm_start:
            logger.info("Allocating contiguous memory of length %d for Ps, and of length %d for Qs.",
                        plan.total_p, plan.total_q)
        state.p_memory_dict[bidx] = torch.empty(plan.total_p, device=device, dtype=dtype)
        state.q_memory_dict[bidx] = torch.empty(plan.total_q, device=device, dtype=dtype)
    pmem, qmem = state.p_memory_dict[bidx], state.q_memory_dict[bidx]
    ps = [pmem[e.p_off : e.p_off + e.n * e.r].view(e.n, e.r) for e in plan.mats]
    qs = [qmem[e.q_off : e.q_off + e.m * e.r].view(e.m, e.r) for e in plan.mats]

    if fresh:
        _random_q_cpu(state, qs)
    for q in qs:
        ref.gram_schmidt_ref(q, state.orthogonalization_epsilon)

    for mat, q, p in zip(mats, qs, ps):
        torch.matmul(mat, q, out=p)

    _allreduce_sum(unc, group)
    unc.div_(ws)
    for s in plan.segs:
        buf[s.g_off : s.g_off + s.numel].copy_(unc[s.dst_off : s.dst_off + s.numel])

    _allreduce_sum(pmem, group)            # summed, not averaged: P is orthogonalised next
    for p in ps:
        ref.gram_schmidt_ref(p, state.orthogonalization_epsilon)
    for mat, p, q in zip(mats, ps, qs):
        torch.matmul(mat.t(), p, out=q)
    _allreduce_sum(qmem, group)
    qmem.div_(ws)
    for p, q, mat in zip(ps, qs, mats):
        torch.matmul(p, q.t(), out=mat)

    if dense_ef:
        state.error_dict[bidx] = buf_copy.sub_(buf)
    elif conef:
        for cnt, (mat, cp) in enumerate(zip(mats, copies)):
            cp.sub_(mat)
            state.error_dict[bidx][cnt].update(cp, beta)

    if not state.warm_start:
        state.p_memory_dict.clear()
        state.q_memory_dict.clear()
    state.maybe_increase_iter(bucket)
    return _done(buf)


def _native_ok(state, buf) -> bool:
    return native.use_native(buf) and buf.dtype == torch.float32


@_measurable
def powerSGD_hook(state: PowerSGDState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Layer-wise PowerSGD with optional (compressed) error feedback."""
    group = _group(state)
    buf = bucket.buffer()
    if state.in_warmup(state.start_powerSGD_iter, bucket):
        state.maybe_increase_iter(bucket)
        return allreduce_fut(group, buf)
    if _native_ok(state, buf):
        from .engine import run_powersgd_native
        return run_powersgd_native(state, bucket, group, variant="powersgd")
    return _powersgd_torch(state, bucket, group)


def hpowerSGD_hook(state: hPowerSGDState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """PowerSGD whose per-matrix error memory is re-compressed after every step
    (top-k as in the reference, or low-rank factors)."""
    return powerSGD_hook(state, bucket)


@_measurable
def C2CS_hook_v2(state: PowerSGDState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """PowerSGD + count sketch built over the ``(m, n)`` reinterpretation of each
    ``(n, m)`` matrix's memory (communication/powerSGD_hook.py:918-920)."""
    group = _group(state)
    buf = bucket.buffer()
    if state.in_warmup(state.start_powerSGD_iter, bucket):
        state.maybe_increase_iter(bucket)
        return allreduce_fut(group, buf)
    if _native_ok(state, buf):
        from .engine import run_powersgd_native
        return run_powersgd_native(state, bucket, group, variant="c2cs")
    return _powersgd_torch(state, bucket, group, transposed_sketch=True)


@_measurable
def batched_powerSGD_hook(state: PowerSGDState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """The whole bucket as one zero-padded square matrix; dense error feedback only."""
    group = _group(state)
    buf = bucket.buffer()
    if state.in_warmup(state.start_powerSGD_iter, bucket):
        state.maybe_increase_iter(bucket)
        return allreduce_fut(group, buf)
    if _native_ok(state, buf):
        from .engine import run_powersgd_native
        return run_powersgd_native(state, bucket, group, variant="batched")
    return _batched_torch(state, bucket, group)


def _batched_torch(state, bucket, group):
    ws = group.size()
    buf = bucket.buffer()
    device, dtype = buf.device, buf.dtype
    bidx = bucket.index()
    total = buf.numel()
    side = math.ceil(math.sqrt(total))
    rank = min(side, state.matrix_approximation_rank)
    state.total_numel_before_compression += total
    state.total_numel_after_compression += side * state.matrix_approximation_rank * 2
    state.account_wire(side * state.matrix_approximation_rank * 2, total, bucket)
    _report_compression_stats(bucket, state)

    padded = torch.zeros(side * side, device=device, dtype=dtype)
    padded[:total].copy_(buf)
    padded_copy = None
    if state.use_error_feedback:
        if bidx in state.error_dict and state.error_dict[bidx].numel() == side * side:
            padded.add_(state.error_dict[bidx])
        else:
            state.error_dict[bidx] = torch.zeros(side * side, device=device, dtype=dtype)
        padded_copy = padded.clone()
    matrix = padded.view(side, side)

    fresh = (not state.warm_start) or bidx not in state.p_memory_dict
    if fresh:
        state.p_memory_dict[bidx] = torch.empty(side * rank, device=device, dtype=dtype)
        state.q_memory_dict[bidx] = torch.empty(side * rank, device=device, dtype=dtype)
    p = state.p_memory_dict[bidx].view(side, rank)
    q = state.q_memory_dict[bidx].view(side, rank)
    if fresh:
        _random_q_cpu(state, [q])
    ref.gram_schmidt_ref(q, state.orthogonalization_epsilon)
    torch.matmul(matrix, q, out=p)
    _allreduce_sum(state.p_memory_dict[bidx], group)
    ref.gram_schmidt_ref(p, state.orthogonalization_epsilon)
    torch.matmul(matrix.t(), p, out=q)
    _allreduce_sum(state.q_memory_dict[bidx], group)
    state.q_memory_dict[bidx].div_(ws)
    torch.matmul(p, q.t(), out=matrix)
    if state.use_error_feedback:
        state.error_dict[bidx] = padded_copy.sub_(padded)
    if not state.warm_start:
        state.p_memory_dict.clear()
        state.q_memory_dict.clear()
    buf.copy_(padded[:total])
    state.maybe_increase_iter(bucket)
    return _done(buf)


# --------------------------------------------------------------------------
# unbiased random-projection compressor
# --------------------------------------------------------------------------
@_measurable
def UnbiasedMtrx_hook(state: unbiasedMtrxState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """``M_hat = mean_ranks(M Q) Q^T`` with a fresh shared Gaussian ``Q`` every step;
    no orthogonalisation, no error feedback, nothing kept between steps.

    The reference also all-reduces ``Q`` although it is identical on every rank
    (communication/unbiasedMtrx_hook.py:279-285); that collective is dropped."""
    group = _group(state)
    buf = bucket.buffer()
    if state.in_warmup(state.start_powerSGD_iter, bucket):
        state.maybe_increase_iter(bucket)
        return allreduce_fut(group, buf)
    if _native_ok(state, buf):
        from .engine import run_powersgd_native
        return run_powersgd_native(state, bucket, group, variant="unbiased")
    ws = group.size()
    device, dtype = buf.device, buf.dtype
    plan = planlib.build_powersgd_plan(buf, bucket.gradients(), state.matrix_approximation_rank,
                                       state.min_compression_rate)
    state.total_numel_before_compression += plan.numel_before
    state.total_numel_after_compression += plan.numel_after
    state.account_wire(plan.numel_after, plan.numel_before, bucket)
    mats = [buf[e.g_off : e.g_off + e.numel].view(e.n, e.m) for e in plan.mats]
    unc = (torch.cat([buf[s.g_off : s.g_off + s.numel] for s in plan.segs])
           if plan.segs else torch.empty(0, device=device, dtype=dtype))
    pmem = torch.empty(plan.total_p, device=device, dtype=dtype)
    qmem = torch.empty(plan.total_q, device=device, dtype=dtype)
    ps = [pmem[e.p_off : e.p_off + e.n * e.r].view(e.n, e.r) for e in plan.mats]
    qs = [qmem[e.q_off : e.q_off + e.m * e.r].view(e.m, e.r) for e in plan.mats]
    _random_q_cpu(state, qs)
    for mat, q, p in zip(mats, qs, ps):
        torch.matmul(mat, q, out=p)
    _allreduce_sum(unc, group)
    unc.div_(ws)
    for s in plan.segs:
        buf[s.g_off : s.g_off + s.numel].copy_(unc[s.dst_off : s.dst_off + s.numel])
    _allreduce_sum(pmem, group)
    pmem.div_(ws)
    for p, q, mat in zip(ps, qs, mats):
        torch.matmul(p, q.t(), out=mat)
    state.maybe_increase_iter(bucket)
    return _done(buf)


# --------------------------------------------------------------------------
# random block
# --------------------------------------------------------------------------
def _draw_starts(state, plan) -> List[int]:
    """One shared-RNG draw per compressed tensor, in bucket order
    (communication/RandomBlock_hook.py:218)."""
    return [int(state.rng.choice(b.numel)) for b in plan.blocks]


def _block_slices(b, start):
    """Flat index ranges of a wrap-around block: [(lo, hi), ...]."""
    end = min(start + b.block, b.numel)
    rest = b.block - (end - start)
    return [(start, end)] + ([(0, rest)] if rest > 0 else [])


def _randblock_torch(state, bucket, group, *, unbiased: bool) -> torch.futures.Future[torch.Tensor]:
    ws = group.size()
    buf = bucket.buffer()
    device, dtype = buf.device, buf.dtype
    bidx = bucket.index()
    plan = planlib.build_block_plan(buf, bucket.gradients(), state.compression_ratio)
    use_ef = (not unbiased) and state.use_error_feedback
    conef = use_ef and state.use_error_compression
    tens = [buf[b.g_off : b.g_off + b.numel] for b in plan.blocks]

    if use_ef:
        errs = state.error_dict.setdefault(bidx, [])
        for cnt, (b, t) in enumerate(zip(plan.blocks, tens)):
            if len(errs) <= cnt:
                if conef:
                    errs.append(make_error_compressor(state.error_compressor, b.n, b.m,
                                                      sketch_size=state.sketch_size,
                                                      seed=state.hash_seed, device=device))
                else:
                    errs.append(torch.zeros(b.n, b.m, device=device, dtype=dtype))
            if conef:
                errs[cnt].query(t, 1.0 - state.beta)
            else:
                t.add_(errs[cnt].view(-1))
                errs[cnt] = t.clone().view(b.n, b.m)

    unc = (torch.cat([buf[s.g_off : s.g_off + s.numel] for s in plan.segs])
           if plan.segs else torch.empty(0, device=device, dtype=dtype))
    if bidx not in state.compressed_tensor_memory or \
            state.compressed_tensor_memory[bidx].numel() != plan.total_block:
        state.compressed_tensor_memory[bidx] = torch.empty(plan.total_block, dtype=torch.float32, device=device)
    staging = state.compressed_tensor_memory[bidx]
    state.account_wire(plan.total_unc + plan.total_block, buf.numel(), bucket)

    starts = _draw_starts(state, plan)
    for cnt, (b, t, start) in enumerate(zip(plan.blocks, tens, starts)):
        pos = b.stage_off
        pieces = _block_slices(b, start)
        for lo, hi in pieces:
            staging[pos : pos + hi - lo].copy_(t[lo:hi])
            pos += hi - lo
        if unbiased:
            staging[b.stage_off : b.stage_off + b.block].div_(b.block / b.numel)
        if use_ef:
            if conef:
                cp = t.clone()
                for lo, hi in pieces:
                    cp[lo:hi].zero_()
                state.error_dict[bidx][cnt].update(cp, state.beta)
            else:
                e = state.error_dict[bidx][cnt].view(-1)
                for lo, hi in pieces:
                    e[lo:hi].zero_()

    _allreduce_sum(unc, group)
    unc.div_(ws)
    for s in plan.segs:
        buf[s.g_off : s.g_off + s.numel].copy_(unc[s.dst_off : s.dst_off + s.numel])
    _allreduce_sum(staging, group)
    staging.div_(ws)
    for b, t, start in zip(plan.blocks, tens, starts):
        t.zero_()
        pos = b.stage_off
        for lo, hi in _block_slices(b, start):
            t[lo:hi].copy_(staging[pos : pos + hi - lo])
            pos += hi - lo
    state.maybe_increase_iter(bucket)
    return _done(buf)


@_measurable
def RandomBlock_hook(state: RandomBlockState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Send one random contiguous block per tensor; the rest goes to error feedback."""
    group = _group(state)
    buf = bucket.buffer()
    if state.in_warmup(state.start_compression_iter, bucket):
        state.maybe_increase_iter(bucket)
        return allreduce_fut(group, buf)
    if _native_ok(state, buf):
        from .engine import run_randblock_native
        return run_randblock_native(state, bucket, group, unbiased=False)
    return _randblock_torch(state, bucket, group, unbiased=False)


@_measurable
def UnbiasedRandomBlock_hook(state: UnbiasedRandomBlockState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Random block without error feedback; selected values are divided by the
    selection probability so the estimate is unbiased."""
    group = _group(state)
    buf = bucket.buffer()
    if state.in_warmup(state.start_compression_iter, bucket):
        state.maybe_increase_iter(bucket)
        return allreduce_fut(group, buf)
    if _native_ok(state, buf):
        from .engine import run_randblock_native
        return run_randblock_native(state, bucket, group, unbiased=True)
    return _randblock_torch(state, bucket, group, unbiased=True)
