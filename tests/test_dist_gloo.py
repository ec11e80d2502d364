"""Multi-process CPU tests over gloo: real DDP hook path, cross-rank consistency,
agreement with an explicit all-gather formula, host-side failure detection."""
import argparse
import datetime
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.nn as nn

import conef_b200 as cb
from conef_b200.ops import reference as ref
from conef_b200.parallel import plan as planlib

from helpers import FakeBucket, free_port, run_ranks

SHAPES = [(24, 3, 3, 3), (24,), (40, 24, 3, 3), (40,), (10, 40), (10,)]


def _ns(name, **kw):
    ns = argparse.Namespace(grad_reducer=name, start_compression_iter=3, compression_ratio=0.1, beta=0.9,
                            sketch_size=0.1, matrix_approximation_rank=2, min_compression_rate=2,
                            orthogonalization_epsilon=0, error_compressor=None)
    for k, v in kw.items():
        setattr(ns, k, v)
    return ns


def _ddp_worker(rank, world, cases):
    for name, err in cases:
        _ddp_case(rank, world, name, err)


def _ddp_case(rank, world, name, err):
    from torch.nn.parallel import DistributedDataParallel as DDP

    torch.manual_seed(0)
    net = nn.Sequential(nn.Conv2d(3, 16, 3, padding=1), nn.ReLU(), nn.Conv2d(16, 32, 3, padding=1), nn.ReLU(),
                        nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(32, 10))
    ddp = DDP(net, bucket_cap_mb=0.01)       # several buckets
    state = cb.get_comm_hooks(_ns(name, error_compressor=err), ddp, None)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05, momentum=0.9)
    torch.manual_seed(100 + rank)
    losses = []
    for _ in range(7):
        x, y = torch.randn(8, 3, 16, 16), torch.randint(0, 10, (8,))
        loss = nn.functional.cross_entropy(ddp(x), y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    flat = torch.cat([p.detach().view(-1) for p in net.parameters()])
    both = [torch.zeros_like(flat) for _ in range(world)]
    dist.all_gather(both, flat)
    for other in both[1:]:
        assert torch.equal(both[0], other), f"{name}: parameters diverged across ranks"
    assert np.isfinite(losses).all()
    if state is not None:
        assert state.iter == 7


_CASES = [(n, None) for n in cb.REDUCERS] + [("conef_powersgd", "count_sketch3"), ("conef_randomblock", "quant8"),
                                             ("hefsgd_powersgd", "lowrank"), ("conef_powersgd", "half_count_sketch")]


@pytest.mark.parametrize("chunk", [0, 1])
def test_ddp_hook_all_ranks_agree(chunk):
    """Every reducer name of the registry (and the extra error compressors) through real DDP."""
    run_ranks(_ddp_worker, world=2, args=(_CASES[chunk::2],), timeout=600)


def _formula_worker(rank, world):
    """ef_powersgd at step 1 equals the closed form computed from all ranks' gradients."""
    s = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2, warm_start=True)
    s.iter = 2
    b = FakeBucket(SHAPES, seed=10 + rank)
    local = b.buffer().clone()
    allb = [torch.zeros_like(local) for _ in range(world)]
    dist.all_gather(allb, local)
    out = cb.powerSGD_hook(s, b).wait()
    plan = planlib.build_powersgd_plan(local, FakeBucket(SHAPES).gradients(), 2, 2)
    mean = sum(allb) / world
    for seg in plan.segs:
        torch.testing.assert_close(out[seg.g_off : seg.g_off + seg.numel], mean[seg.g_off : seg.g_off + seg.numel])
    # replay Q init: same shared seed on every rank
    rng = np.random.RandomState(0)
    with torch.random.fork_rng(devices=[]):
        torch.manual_seed(int(rng.randint(1_000_000_000)))
        qs = [torch.randn(e.m, e.r) for e in plan.mats]
    for e, q in zip(plan.mats, qs):
        ref.gram_schmidt_ref(q)
        mats = [a[e.g_off : e.g_off + e.numel].view(e.n, e.m) for a in allb]
        p = sum(m @ q for m in mats)                      # summed, not averaged
        ref.gram_schmidt_ref(p)
        q2 = sum(m.t() @ p for m in mats) / world         # averaged
        torch.testing.assert_close(out[e.g_off : e.g_off + e.numel].view(e.n, e.m), p @ q2.t(), atol=1e-5, rtol=1e-4)
    # error memory is local input minus the shared output (also for uncompressed tensors)
    torch.testing.assert_close(s.error_dict[0], local - out)


def test_powersgd_matches_closed_form_ws2():
    run_ranks(_formula_worker, world=2)


def test_powersgd_matches_closed_form_ws4():
    run_ranks(_formula_worker, world=4)


def _randblock_formula_worker(rank, world):
    s = cb.RandomBlockState(None, start_compression_iter=2, compression_ratio=0.2, use_error_feedback=True)
    s.iter = 2
    b = FakeBucket(SHAPES, seed=20 + rank)
    local = b.buffer().clone()
    allb = [torch.zeros_like(local) for _ in range(world)]
    dist.all_gather(allb, local)
    out = cb.RandomBlock_hook(s, b).wait()
    mean = sum(allb) / world
    bp = planlib.build_block_plan(local, FakeBucket(SHAPES).gradients(), 0.2)
    rng = np.random.RandomState(42)
    for blk in bp.blocks:
        mask = ref.block_mask(blk.numel, 0.2, int(rng.choice(blk.numel)))
        t = out[blk.g_off : blk.g_off + blk.numel]
        torch.testing.assert_close(t[mask], mean[blk.g_off : blk.g_off + blk.numel][mask])
        assert float(t[~mask].abs().sum()) == 0.0
    for seg in bp.segs:
        torch.testing.assert_close(out[seg.g_off : seg.g_off + seg.numel], mean[seg.g_off : seg.g_off + seg.numel])


def test_randomblock_matches_closed_form():
    run_ranks(_randblock_formula_worker, world=2)


def _resume_worker(rank, world):
    """Checkpoint after two compressed steps, restore into a fresh state, next step identical."""
    import pickle

    def fresh():
        s = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2, use_error_compression=True,
                             sketch_size=0.2, error_compressor="count_sketch3", hash_seed=5)
        s.iter = 2
        return s
    a = fresh()
    b = FakeBucket(SHAPES, seed=rank)
    for i in range(2):
        b.refill(50 + 10 * i + rank)
        cb.powerSGD_hook(a, b).wait()
    blob = pickle.dumps(a.state_dict())
    b.refill(999 + rank)
    want = cb.powerSGD_hook(a, b).wait().clone()
    r = fresh()
    r.load_state_dict(pickle.loads(blob), device="cpu")
    b2 = FakeBucket(SHAPES, seed=rank)
    b2.refill(999 + rank)
    got = cb.powerSGD_hook(r, b2).wait()
    assert torch.equal(want, got)


def test_resume_mid_run_ws2():
    run_ranks(_resume_worker, world=2)


# ---- failure detection, made on the host ------------------------------------
def _failing_rank(rank, port, outq):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=8))
    s = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2)
    s.iter = 2
    b = FakeBucket(SHAPES, seed=rank)
    cb.powerSGD_hook(s, b).wait()                      # a healthy step first
    if rank == 1:
        outq.put(("rank1", "leaving"))
        os._exit(0)                                    # dies between steps, never joins the next collective
    try:
        b.refill(3)
        cb.powerSGD_hook(s, b).wait()
        outq.put(("rank0", "no error"))
    except Exception as exc:  # noqa: BLE001
        outq.put(("rank0", f"detected: {type(exc).__name__}"))
    os._exit(0)


def test_peer_exit_is_detected_not_hung():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_failing_rank, args=(r, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
    assert not any(p.is_alive() for p in procs), "a rank hung after its peer left"
    msgs = {}
    while not q.empty():
        k, v = q.get()
        msgs[k] = v
    assert msgs.get("rank1") == "leaving"
    assert msgs.get("rank0", "").startswith("detected"), msgs
