"""Pure-CPU unit tests: compression decision, Gram-Schmidt, blocks, states."""
import argparse
import pickle

import numpy as np
import pytest
import torch

import conef_b200 as cb
from conef_b200.ops import reference as ref
from conef_b200.parallel import plan as planlib

from helpers import FakeBucket


def test_should_compress_truth_table():
    # compress iff (n + m) * r * min_rate < n * m
    assert ref.should_compress(640, 5760, 4, 2) == (True, 640 * 5760, 6400 * 4)
    assert ref.should_compress(10, 10, 4, 2)[0] is False       # 160 < 100 false
    assert ref.should_compress(16, 27, 2, 2)[0] is True        # 172 < 432
    assert ref.should_compress(100, 1, 1, 2)[0] is False       # vectors never pay off at rate 2
    assert ref.should_compress(100, 1, 1, 0.5)[0] is True


def test_gram_schmidt_orthonormal_and_eps():
    torch.manual_seed(0)
    a = torch.randn(200, 6)
    ref.gram_schmidt_ref(a)
    torch.testing.assert_close(a.t() @ a, torch.eye(6), atol=1e-5, rtol=0)
    z = torch.zeros(10, 2)
    ref.gram_schmidt_ref(z, eps=1e-8)
    assert torch.isfinite(z).all()


def test_block_wraparound():
    block, first, rest = ref.block_bounds(100, 0.1, 95)
    assert (block, first, rest) == (10, 5, 5)
    mask = ref.block_mask(100, 0.1, 95)
    assert mask.sum() == 10 and mask[95:].all() and mask[:5].all()
    assert ref.block_bounds(5, 0.01, 4) == (1, 1, 0)


def test_plan_partition_and_offsets():
    b = FakeBucket([(64, 3, 3, 3), (64,), (128, 64, 3, 3), (10, 128), (10,)])
    plan = planlib.build_powersgd_plan(b.buffer(), b.gradients(), 4, 2)
    assert [(e.n, e.m, e.r) for e in plan.mats] == [(64, 27, 4), (128, 576, 4), (10, 128, 4)]
    assert [(e.p_off, e.q_off) for e in plan.mats] == [(0, 0), (256, 108), (768, 2412)]
    total = sum(e.numel for e in plan.mats) + sum(s.numel for s in plan.segs)
    assert total == b.buffer().numel()
    offs = planlib.grad_offsets(b.buffer(), b.gradients())
    assert offs == [0, 1728, 1792, 1792 + 73728, 1792 + 73728 + 1280]
    bp = planlib.build_block_plan(b.buffer(), b.gradients(), 0.1)
    assert [x.block for x in bp.blocks] == [172, 7372, 128]
    assert bp.total_unc == 74


def test_state_ctor_validation():
    with pytest.raises(ValueError):
        cb.PowerSGDState(None, start_powerSGD_iter=1)
    cb.PowerSGDState(None, start_powerSGD_iter=1, use_error_feedback=False, warm_start=False)
    with pytest.raises(ValueError):
        cb.RandomBlockState(None, start_compression_iter=1)
    with pytest.raises(ValueError):
        cb.RandomBlockState(None, use_error_compression=True, use_error_feedback=False)
    with pytest.raises(ValueError):
        cb.UnbiasedRandomBlockState(None, start_compression_iter=0)
    with pytest.raises(ValueError):
        cb.PowerSGDState(None, error_compressor="nope")


def test_state_defaults_match_reference_layout():
    s = cb.PowerSGDState(None)
    assert (s.matrix_approximation_rank, s.start_powerSGD_iter, s.min_compression_rate) == (1, 1000, 2)
    assert (s.beta, s.sketch_size, s.use_error_feedback, s.warm_start, s.use_error_compression) == \
        (0.9, 0.5, True, True, False)
    assert isinstance(s.rng, np.random.RandomState) and s.iter == 0
    r = cb.RandomBlockState(None)
    assert (r.compression_ratio, r.start_compression_iter) == (0.1, 1000)
    assert int(cb.RandomBlockState(None).rng.randint(10 ** 9)) == int(np.random.RandomState(42).randint(10 ** 9))
    u = cb.unbiasedMtrxState(None)
    assert int(u.rng.randint(10 ** 9)) == int(np.random.RandomState(421).randint(10 ** 9))
    h = cb.hPowerSGDState(None)
    assert h.topk_ratio == 0.4


def test_state_pickle_drops_process_group_and_caches():
    s = cb.PowerSGDState("not-picklable-group", start_powerSGD_iter=5)
    s.error_dict[0] = torch.ones(4)
    s.iter = 7
    s._engines[0] = object()
    t = pickle.loads(pickle.dumps(s))
    assert t.process_group is None and t._engines == {} and t.iter == 7
    assert torch.equal(t.error_dict[0], torch.ones(4))


def test_registry_names():
    ns = argparse.Namespace(start_compression_iter=10, compression_ratio=0.1, beta=0.9, sketch_size=0.2,
                            matrix_approximation_rank=4, min_compression_rate=2, orthogonalization_epsilon=0)
    kinds = {}
    for name in cb.REDUCERS:
        ns.grad_reducer = name
        state, hook = cb.build_state_and_hook(ns)
        kinds[name] = (type(state).__name__ if state is not None else None, getattr(hook, "__name__", None))
    assert kinds["allreduce"] == (None, None)
    assert kinds["conef_powersgd"] == ("PowerSGDState", "powerSGD_hook")
    assert kinds["hefsgd_powersgd"] == ("hPowerSGDState", "hpowerSGD_hook")
    assert kinds["ef_randomblock"] == ("RandomBlockState", "RandomBlock_hook")
    assert kinds["unbiased_randomblock"] == ("UnbiasedRandomBlockState", "UnbiasedRandomBlock_hook")
    assert kinds["unbiased_mtrx"] == ("unbiasedMtrxState", "UnbiasedMtrx_hook")
    ns.grad_reducer = "bogus"
    with pytest.raises(ValueError):
        cb.build_state_and_hook(ns)


def test_reference_import_names():
    import communication.powerSGD_hook as powerSGD
    import communication.RandomBlock_hook as RandomBlock
    from communication.compressors.CountSketch import DenseCS
    from communication.compressors.halfCountSketch import DenseCS as HalfCS

    assert powerSGD.PowerSGDState is cb.PowerSGDState and powerSGD.powerSGD_hook is cb.powerSGD_hook
    assert RandomBlock.RandomBlock_hook is cb.RandomBlock_hook
    assert DenseCS(2, 10, 0.5, device="cpu").cs.dtype == torch.float32
    assert HalfCS(2, 10, 0.5, device="cpu").cs.dtype == torch.float16


# ---- hooks on a single rank through fake buckets ---------------------------
SHAPES = [(32, 3, 3, 3), (32,), (48, 32, 3, 3), (48,), (10, 48), (10,)]


def _run(hook, state, bucket, steps=1):
    for i in range(steps):
        if i:
            bucket.refill(100 + i)
        out = hook(state, bucket).wait()
    return out


def test_warmup_is_plain_allreduce_and_iter_counts(single_rank_group):
    s = cb.PowerSGDState(None, start_powerSGD_iter=3, matrix_approximation_rank=2)
    b = FakeBucket(SHAPES, last=False)
    before = b.buffer().clone()
    cb.powerSGD_hook(s, b).wait()
    assert torch.equal(b.buffer(), before) and s.iter == 0     # not the last bucket: no increment
    b2 = FakeBucket(SHAPES, last=True)
    cb.powerSGD_hook(s, b2).wait()
    assert s.iter == 1


def test_powersgd_single_rank_math(single_rank_group):
    s = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2, use_error_feedback=True)
    s.iter = 2
    b = FakeBucket(SHAPES)
    g0 = b.buffer().clone()
    out = cb.powerSGD_hook(s, b).wait()
    assert out is b.buffer()
    plan = planlib.build_powersgd_plan(g0, FakeBucket(SHAPES).gradients(), 2, 2)
    # uncompressed tensors are untouched at world size 1, compressed ones are rank-2
    for seg in plan.segs:
        assert torch.equal(out[seg.g_off : seg.g_off + seg.numel], g0[seg.g_off : seg.g_off + seg.numel])
    for e in plan.mats:
        m = out[e.g_off : e.g_off + e.numel].view(e.n, e.m)
        assert torch.linalg.matrix_rank(m) <= 2
        q = s.q_memory_dict[0][e.q_off : e.q_off + e.m * e.r].view(e.m, e.r)
        p = s.p_memory_dict[0][e.p_off : e.p_off + e.n * e.r].view(e.n, e.r)
        torch.testing.assert_close(p.t() @ p, torch.eye(e.r), atol=1e-5, rtol=0)
        torch.testing.assert_close(p @ q.t(), m, atol=1e-5, rtol=1e-5)
    # dense error = input - output
    torch.testing.assert_close(s.error_dict[0], g0 - out)
    rate, before, after = s.compression_stats()
    assert before == g0.numel() and rate > 1


def test_conef_error_memory_is_smaller_and_feeds_back(single_rank_group):
    dense = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2)
    conef = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2, use_error_compression=True,
                             sketch_size=0.1)
    dense.iter = conef.iter = 2
    _run(cb.powerSGD_hook, dense, FakeBucket(SHAPES), 2)
    _run(cb.powerSGD_hook, conef, FakeBucket(SHAPES), 2)
    assert conef.ef_buffer_bytes() < 0.15 * dense.ef_buffer_bytes()
    assert all(float(c.cs.abs().sum()) > 0 for c in conef.error_dict[0].values())


def test_randomblock_zero_outside_block(single_rank_group):
    s = cb.RandomBlockState(None, start_compression_iter=2, compression_ratio=0.1)
    s.iter = 2
    b = FakeBucket(SHAPES)
    g0 = b.buffer().clone()
    out = cb.RandomBlock_hook(s, b).wait()
    bp = planlib.build_block_plan(g0, FakeBucket(SHAPES).gradients(), 0.1)
    rng = np.random.RandomState(42)
    for blk in bp.blocks:
        start = int(rng.choice(blk.numel))
        mask = ref.block_mask(blk.numel, 0.1, start)
        t = out[blk.g_off : blk.g_off + blk.numel]
        assert torch.equal(t[~mask], torch.zeros_like(t[~mask]))
        assert torch.equal(t[mask], g0[blk.g_off : blk.g_off + blk.numel][mask])
        err = s.error_dict[0][bp.blocks.index(blk)].view(-1)
        assert torch.equal(err[mask], torch.zeros_like(err[mask]))
        assert torch.equal(err[~mask], g0[blk.g_off : blk.g_off + blk.numel][~mask])


def test_unbiased_randomblock_scaling(single_rank_group):
    s = cb.UnbiasedRandomBlockState(None, start_compression_iter=2, compression_ratio=0.25)
    s.iter = 2
    b = FakeBucket([(16, 16)])
    g0 = b.buffer().clone()
    out = cb.UnbiasedRandomBlock_hook(s, b).wait()
    nz = out != 0
    assert int(nz.sum()) == 64
    torch.testing.assert_close(out[nz], g0[nz] * 4.0)


def test_unbiased_mtrx_and_batched_and_c2cs_run(single_rank_group):
    u = cb.unbiasedMtrxState(None, start_powerSGD_iter=2, matrix_approximation_rank=4)
    u.iter = 2
    out = cb.UnbiasedMtrx_hook(u, FakeBucket(SHAPES)).wait()
    assert torch.isfinite(out).all() and u.p_memory_dict == {}
    bt = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=1)
    bt.iter = 2
    b = FakeBucket(SHAPES)
    n = b.buffer().numel()
    out = cb.batched_powerSGD_hook(bt, b).wait()
    assert out.numel() == n and torch.isfinite(out).all()
    assert bt.error_dict[0].numel() == int(np.ceil(np.sqrt(n))) ** 2
    c2 = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2, use_error_compression=True,
                          sketch_size=0.2)
    c2.iter = 2
    cb.C2CS_hook_v2(c2, FakeBucket(SHAPES)).wait()
    comp = c2.error_dict[0][0]
    assert (comp.N, comp.D) == (27, 32)          # sketch over the (m, n) reinterpretation of the 32x27 matrix


@pytest.mark.parametrize("kind", ["count_sketch", "count_sketch3", "half_count_sketch", "topk", "quant8", "lowrank"])
def test_every_error_compressor_with_powersgd(single_rank_group, kind):
    s = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2, use_error_compression=True,
                         sketch_size=0.2, error_compressor=kind, error_rank=2)
    s.iter = 2
    out = _run(cb.powerSGD_hook, s, FakeBucket(SHAPES), 3)
    assert torch.isfinite(out).all() and s.ef_buffer_bytes() > 0


def test_state_dict_resume_is_bit_exact(single_rank_group):
    def fresh():
        s = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2, use_error_compression=True,
                             sketch_size=0.2)
        s.iter = 2
        return s
    a = fresh()
    b = FakeBucket(SHAPES)
    _run(cb.powerSGD_hook, a, b, 2)
    saved = pickle.loads(pickle.dumps(a.state_dict()))       # as torch.save / load would do
    b.refill(555)
    want = cb.powerSGD_hook(a, b).wait().clone()
    r = fresh()
    r.load_state_dict(saved, device="cpu")
    b2 = FakeBucket(SHAPES)
    b2.refill(555)
    got = cb.powerSGD_hook(r, b2).wait()
    assert torch.equal(want, got)
    assert r.iter == a.iter


def test_randomblock_resume_is_bit_exact(single_rank_group):
    def fresh():
        s = cb.RandomBlockState(None, start_compression_iter=2, use_error_compression=True, sketch_size=0.2)
        s.iter = 2
        return s
    a = fresh()
    b = FakeBucket(SHAPES)
    _run(cb.RandomBlock_hook, a, b, 2)
    saved = pickle.loads(pickle.dumps(a.state_dict()))
    b.refill(9)
    want = cb.RandomBlock_hook(a, b).wait().clone()
    r = fresh()
    r.load_state_dict(saved, device="cpu")
    b2 = FakeBucket(SHAPES)
    b2.refill(9)
    assert torch.equal(want, cb.RandomBlock_hook(r, b2).wait())


def test_wire_bytes_per_step_matches_the_plan(single_rank_group):
    """What a compressed step puts on the wire: P + Q + uncompressed tensors for PowerSGD,
    blocks + uncompressed tensors for RandomBlock."""
    import conef_b200 as cb
    from conef_b200.parallel import plan as planlib
    shapes = [(64, 48), (48,), (32, 16, 3, 3), (5,)]
    b = FakeBucket(shapes)
    s = cb.PowerSGDState(None, matrix_approximation_rank=2, start_powerSGD_iter=2)
    s.iter = 2
    assert s.wire_bytes_per_step() == 0.0
    for _ in range(3):
        cb.powerSGD_hook(s, b).wait()
    plan = planlib.build_powersgd_plan(b.buffer(), b.gradients(), 2, 2)
    assert s.wire_bytes_per_step() == 4.0 * plan.numel_after
    assert s.wire_bytes_per_step() == 4.0 * (plan.total_p + plan.total_q + plan.total_unc)
    assert abs(s.wire_compression_rate() - s.compression_stats()[0]) < 1e-9
    r = cb.RandomBlockState(None, compression_ratio=0.1, start_compression_iter=2)
    r.iter = 2
    for _ in range(2):
        cb.RandomBlock_hook(r, b).wait()
    sent = sum(max(1, int(0.1 * n)) for n in (64 * 48, 32 * 16 * 9)) + 48 + 5
    assert r.wire_bytes_per_step() == 4.0 * sent
    # the counters are run-time only: a restored state starts counting again
    s2 = cb.PowerSGDState(None, matrix_approximation_rank=2, start_powerSGD_iter=2)
    s2.load_state_dict(s.state_dict(), device="cpu")
    assert s2.wire_bytes_per_step() == 0.0


def _nearly_dependent(n, r, relres, seed):
    """(n x r) block whose columns 3 and 6 lie within ``relres`` (relative) of the span of earlier ones."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(n, r, generator=g, dtype=torch.float64)
    a[:, 3] = 0.7 * a[:, 0] - 1.3 * a[:, 1] + relres * torch.randn(n, generator=g, dtype=torch.float64)
    a[:, 6] = a[:, 2] + a[:, 5] + relres * torch.randn(n, generator=g, dtype=torch.float64)
    return a


@pytest.mark.parametrize("relres", [1e-3, 1e-4, 1e-5, 1e-6])
def test_shifted_cholesky_qr_keeps_nearly_dependent_columns_alive(relres):
    """The Gram-matrix orthogonalisation of the native path in fp32: no column is dropped, the
    result is orthonormal, and it spans what Gram-Schmidt in float64 spans."""
    a64 = _nearly_dependent(2000, 8, relres, seed=11)
    a32 = a64.float().clone()
    ref.shifted_cholesky_qr2_(a32)
    q = a32.double()
    assert bool((q.norm(dim=0) > 0.99).all()), q.norm(dim=0)
    torch.testing.assert_close(q.t() @ q, torch.eye(8, dtype=torch.float64), rtol=0, atol=5e-5)
    want = a64.float().double()
    ref.gram_schmidt_ref(want)                         # float64 oracle of the reference's loop
    # same span: the oracle's columns are reproduced by projecting onto ours
    resid = want - q @ (q.t() @ want)
    # the residual direction of a nearly dependent column is only known to (fp32 epsilon / relres)
    assert float(resid.norm(dim=0).max()) < 2e-7 / relres + 1e-4


def test_shifted_cholesky_qr_matches_gram_schmidt_on_conditioned_input():
    torch.manual_seed(5)
    a = torch.randn(700, 6)
    b = a.clone()
    ref.shifted_cholesky_qr2_(a)
    ref.gram_schmidt_ref(b)
    torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("kw", [dict(momentum=0.9, nesterov=True, weight_decay=5e-4), dict(momentum=0.9, dampening=0.1),
                                dict(weight_decay=1e-2), dict()])
def test_fused_sgd_matches_torch_sgd_on_cpu(kw):
    """FusedSGD's PyTorch-ops path (CPU tensors) against torch.optim.SGD over several steps."""
    from conef_b200.optim import FusedSGD
    torch.manual_seed(0)
    ref_p = [torch.nn.Parameter(torch.randn(13, 7)), torch.nn.Parameter(torch.randn(5))]
    own_p = [torch.nn.Parameter(p.detach().clone()) for p in ref_p]
    ref_opt, own_opt = torch.optim.SGD(ref_p, lr=0.1, **kw), FusedSGD(own_p, lr=0.1, **kw)
    for step in range(4):
        for a, b in zip(ref_p, own_p):
            g = torch.randn_like(a)
            a.grad, b.grad = g.clone(), g.clone()
        ref_opt.step()
        own_opt.step()
    for a, b in zip(ref_p, own_p):
        torch.testing.assert_close(a, b)


def test_fused_sgd_zero_grad_keeps_or_drops_the_gradient_tensors():
    """``zero_grad(set_to_none=False)`` clears in place (same tensors, any dtype mix); the default drops them."""
    from conef_b200.optim import FusedSGD
    ps = [torch.nn.Parameter(torch.randn(5, 3)), torch.nn.Parameter(torch.randn(7).double()),
          torch.nn.Parameter(torch.randn(2, 2))]
    opt = FusedSGD(ps, lr=0.1, momentum=0.9)
    for p in ps[:2]:
        p.grad = torch.randn_like(p)
    kept = [p.grad for p in ps[:2]]
    opt.zero_grad(set_to_none=False)
    assert all(p.grad is g and float(g.abs().sum()) == 0 for p, g in zip(ps[:2], kept)) and ps[2].grad is None
    opt.zero_grad()
    assert all(p.grad is None for p in ps)
