"""tcgen05 / TMA tiles for P = M Q and Q = M^T P against fp32 matmul (needs a B200)."""
import pytest
import torch

import conef_b200 as cb
from conef_b200.ops import native
from conef_b200.parallel import plan as planlib
from conef_b200.parallel.engine import PowerSGDEngine

from helpers import FakeBucket

pytestmark = pytest.mark.gpu
DEV = "cuda"
# TMA-addressable matrices (16-byte aligned start, row pitch multiple of 16 bytes) of ragged
# sizes, plus one that is not addressable and must fall back to the SIMT kernel.
SHAPES = [(256, 1024), (64,), (130, 64, 3, 3), (640, 40, 3, 3), (1000, 36), (4,), (3, 5001), (33, 2052)]
# Row pitches that are not a multiple of 16 bytes (the LSTM's 650 columns, a first convolution's 27):
# addressed through the folded view, `fold` rows read as one; (77, 650) has an odd row count for fold 2
# and stays on the SIMT kernels.
SHAPES_FOLD = [(260, 650), (64, 27), (1302, 650), (128, 130), (78, 650), (77, 650), (10,)]
SHAPE_SETS = {"aligned": SHAPES, "folded": SHAPES_FOLD}


def _rel(a, b):
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def _engine(rank, monkeypatch, group, shapes=SHAPES):
    monkeypatch.setenv("CONEF_TC", "1")
    monkeypatch.setenv("CONEF_BACKEND", "native")
    s = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=rank, use_error_feedback=False,
                         warm_start=False)
    b = FakeBucket(shapes, device=DEV, seed=3)
    eng = PowerSGDEngine(s, b.buffer(), b.gradients(), group, "powersgd")
    return eng, b


def _addressable(e, np_cols):
    """TMA needs a 16-byte aligned start and a row pitch that is a multiple of 16 bytes - of the
    matrix itself, or of its folded view (fold rows read as one; needs n % fold == 0 and
    fold * r accumulator columns)."""
    import math
    fold = 4 // math.gcd(e.m, 4)
    folded = fold > 1 and e.n % fold == 0 and fold * e.r <= np_cols
    return e.g_off % 4 == 0 and (e.m % 4 == 0 or folded)


@pytest.mark.parametrize("shapes", ["aligned", "folded"])
@pytest.mark.parametrize("rank", [4, 8, 20])
def test_tc_p_and_q_tiles_match_matmul(single_rank_group, monkeypatch, rank, shapes):
    eng, b = _engine(rank, monkeypatch, single_rank_group, SHAPE_SETS[shapes])
    assert eng.tc_ok.tolist() == [_addressable(e, eng.np_cols) for e in eng.plan.mats]
    if shapes == "folded" and rank == 20:
        assert not any(eng.tc_ok)          # fold * r does not fit the accumulator: everything stays SIMT
        return
    assert eng.use_tc, "tensor-core path should be available on sm_100"
    assert any(eng.tc_ok)
    if shapes == "folded" and rank == 4:
        assert [int(r["fold"]) for r in eng.mats_host] == [2, 4, 2, 2, 2, 1]
    plan = eng.plan
    buf = b.buffer()
    st = native.stream_ptr(buf.device)
    g = torch.Generator().manual_seed(0)
    qmem = torch.randn(plan.total_q, generator=g).to(DEV)
    pmem = torch.zeros(plan.total_p, device=DEV)       # split-K tiles accumulate
    eng._launch_p(buf.data_ptr(), 0, qmem, pmem, st)
    torch.cuda.synchronize()
    assert int(eng.status[0]) == 0, "an mbarrier wait gave up"
    errs = []
    for e in plan.mats:
        m = buf[e.g_off : e.g_off + e.numel].view(e.n, e.m)
        q = qmem[e.q_off : e.q_off + e.m * e.r].view(e.m, e.r)
        want = m.double() @ q.double()
        got = pmem[e.p_off : e.p_off + e.n * e.r].view(e.n, e.r)
        errs.append(("P", e.n, e.m, e.r, _rel(got.double(), want)))
    print(errs)
    assert all(x[-1] < 3e-3 for x in errs), errs
    pmem = torch.cat([(buf[e.g_off : e.g_off + e.numel].view(e.n, e.m) @ qmem[e.q_off : e.q_off + e.m * e.r].view(e.m, e.r)).reshape(-1) for e in plan.mats])
    errs = []
    # Q = M^T P
    qout = torch.zeros(plan.total_q, device=DEV)
    eng._launch_q(buf.data_ptr(), 0, pmem, qout, st)
    torch.cuda.synchronize()
    assert int(eng.status[0]) == 0
    for e in plan.mats:
        m = buf[e.g_off : e.g_off + e.numel].view(e.n, e.m)
        p = pmem[e.p_off : e.p_off + e.n * e.r].view(e.n, e.r)
        want = m.double().t() @ p.double()
        got = qout[e.q_off : e.q_off + e.m * e.r].view(e.m, e.r)
        errs.append(("Q", e.n, e.m, e.r, _rel(got.double(), want)))
    print(errs)
    assert all(x[-1] < 3e-3 for x in errs), errs


@pytest.mark.parametrize("kw", [
    dict(matrix_approximation_rank=4, use_error_feedback=True),
    dict(matrix_approximation_rank=4, use_error_feedback=True, use_error_compression=True, sketch_size=0.1),
], ids=["ef", "conef"])
@pytest.mark.parametrize("shapes", ["aligned", "folded"])
def test_hook_with_tensorcore_path_matches_cpu(single_rank_group, monkeypatch, kw, shapes):
    SHAPES = SHAPE_SETS[shapes]

    def mk(device):
        s = cb.PowerSGDState(None, start_powerSGD_iter=2, **kw)
        s.iter = 2
        fb = FakeBucket(SHAPES)
        plan = planlib.build_powersgd_plan(fb.buffer(), fb.gradients(), 4, 2)
        g = torch.Generator().manual_seed(0)
        s.p_memory_dict[0] = torch.zeros(plan.total_p).to(device)
        s.q_memory_dict[0] = torch.randn(plan.total_q, generator=g).to(device)
        return s

    def run(device, backend, tc):
        monkeypatch.setenv("CONEF_BACKEND", backend)
        monkeypatch.setenv("CONEF_TC", tc)
        s = mk(device)
        b = FakeBucket(SHAPES, device=device, seed=1)
        outs = []
        for i in range(3):
            b.refill(20 + i)
            outs.append(cb.powerSGD_hook(s, b).wait().detach().cpu().clone())
        if device != "cpu":
            torch.cuda.synchronize()
            s.check_status()
            assert s._engines[0].use_tc == (tc == "1")
        return outs
    tc = run(DEV, "native", "1")
    cpu = run("cpu", "torch", "0")
    for a, c in zip(tc, cpu):
        assert _rel(a, c) < 1e-2, _rel(a, c)
