"""Auxiliary subsystems on CPU: checkpoint / resume, graceful stop, tracing, schedulers, data helpers."""
import os
import signal

import numpy as np
import pytest
import torch

import conef_b200 as cb
from conef_b200 import data, optim, utils
from conef_b200.ops import reference as ref

from helpers import FakeBucket

SHAPES = [(32, 3, 3, 3), (32,), (48, 32, 3, 3), (10, 48), (10,)]


def test_resumed_state_waits_for_the_rebuilt_bucket_layout(single_rank_group):
    s = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2)
    s.iter = 2
    b = FakeBucket(SHAPES)
    cb.powerSGD_hook(s, b).wait()
    saved = s.state_dict()
    assert saved["bucket_signatures"][0][0] == b.buffer().numel()
    r = cb.PowerSGDState(None, start_powerSGD_iter=2, matrix_approximation_rank=2)
    r.load_state_dict(saved, device="cpu")
    # first iteration of the new process: DDP still uses its initial bucket assignment
    other = FakeBucket([(10, 48), (10,)], last=True)
    before = other.buffer().clone()
    err_before = r.error_dict[0].clone()
    out = cb.powerSGD_hook(r, other).wait()
    assert torch.equal(out, before) and torch.equal(r.error_dict[0], err_before)      # plain all-reduce, state untouched
    # after the rebuild the saved layout is back and compression resumes
    again = FakeBucket(SHAPES)
    g0 = again.buffer().clone()
    out = cb.powerSGD_hook(r, again).wait()
    assert not torch.equal(out, g0)


def test_checkpoint_roundtrip_keeps_last_three(tmp_path):
    net = torch.nn.Linear(4, 3)
    opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
    state = cb.PowerSGDState(None, start_powerSGD_iter=2)
    state.error_dict[0] = torch.arange(5.0)
    state.iter = 9
    for step in (1, 2, 3, 4, 5):
        utils.save_checkpoint(str(tmp_path), step, model=net, optimizer=opt, reducer_state=state, extra={"epoch": step})
    files = sorted(os.listdir(tmp_path))
    assert files == ["ckpt_3.pt", "ckpt_4.pt", "ckpt_5.pt"]
    assert utils.latest_checkpoint(str(tmp_path)).endswith("ckpt_5.pt")
    net2 = torch.nn.Linear(4, 3)
    st2 = cb.PowerSGDState(None, start_powerSGD_iter=2)
    info = utils.load_checkpoint(utils.latest_checkpoint(str(tmp_path)), model=net2, reducer_state=st2, device="cpu")
    assert info == {"step": 5, "extra": {"epoch": 5}}
    assert torch.equal(net2.weight, net.weight) and st2.iter == 9
    assert torch.equal(st2.error_dict[0], torch.arange(5.0))


def test_graceful_stop_sets_flag_on_sigterm():
    stop = utils.GracefulStop()
    try:
        assert not stop.requested
        os.kill(os.getpid(), signal.SIGTERM)
        assert stop.requested
    finally:
        stop.restore()


def test_phase_timer_and_exposed_comm():
    t = utils.PhaseTimer()
    for _ in range(3):
        with t.phase("work", device="cpu"):
            sum(range(1000))
    s = t.summary()
    assert s["work"]["calls"] == 3 and s["work"]["ms"] >= 0
    assert utils.exposed_comm_ms(12.5, 10.0) == 2.5 and utils.exposed_comm_ms(9.0, 10.0) == 0.0
    assert utils.max_over_ranks(3.0) == 3.0


def test_warmup_schedulers():
    p = [torch.nn.Parameter(torch.zeros(2))]
    for cls, last in ((optim.LinearWarmUpScheduler, 0.0), (optim.ConstantWarmUpScheduler, 1.0),
                      (optim.CosineWarmUpScheduler, 0.0), (optim.PolyWarmUpScheduler, 0.0)):
        o = optim.FusedLAMB(p, lr=1.0)
        s = cls(o, warmup=0.2, total_steps=10)
        lrs = []
        for _ in range(10):
            p[0].grad = torch.ones(2)
            s.step()
            lrs.append(o.param_groups[0]["lr"])
            o.step()
        assert lrs[0] == pytest.approx(0.5) and max(lrs) <= 1.0 + 1e-9
        assert lrs[-1] == pytest.approx(last, abs=1e-6)


def test_bert_adam_matches_manual_step():
    w = torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    o = optim.BertAdam([w], lr=0.1, weight_decay=0.0, max_grad_norm=-1)
    w.grad = torch.tensor([0.5, 0.5])
    o.step()
    m, v = 0.1 * 0.5, 0.001 * 0.25
    torch.testing.assert_close(w.detach(), torch.tensor([1.0, -2.0]) - 0.1 * m / (v ** 0.5 + 1e-6))


def test_data_helpers(tmp_path):
    ids, labels = data.mask_tokens(torch.randint(1000, 30000, (128,)), 30522, generator=torch.Generator().manual_seed(0))
    n = int((labels >= 0).sum())
    assert 1 <= n <= 20 and int((ids == 103).sum()) <= n
    stream = data.synthetic_token_stream(1000, 50)
    a, b = data.batchify(stream, 20, 0, 2), data.batchify(stream, 20, 1, 2)
    assert a.shape == b.shape == (50, 10) and not torch.equal(a, b)
    x, y = data.get_batch(a, 0, 35)
    assert x.shape == (35, 10) and torch.equal(y.view(35, 10), a[1:36])
    (tmp_path / "vocab.txt").write_text("\n".join(["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "un", "##aff", "##able", "hello", ","]))
    tok = data.BertTokenizer(str(tmp_path / "vocab.txt"))
    assert tok.tokenize("Hello, unaffable xyz") == ["hello", ",", "un", "##aff", "##able", "[UNK]"]
    assert tok.convert_ids_to_tokens(tok.convert_tokens_to_ids(["hello", "[MASK]"])) == ["hello", "[MASK]"]
    src, tgt = data.collate_translation([data.SyntheticTranslationPairs(4)[i] for i in range(3)])
    assert src.shape[1] == 3 and int(src[0, 0]) == 2


def test_trainer_checkpoint_resume_over_gloo(single_rank_group, tmp_path):
    import argparse

    import torch.nn.functional as F

    from conef_b200 import DataParallelTrainer, models
    ns = argparse.Namespace(grad_reducer="conef_powersgd", start_compression_iter=2, compression_ratio=0.1, beta=0.9,
                            sketch_size=0.2, matrix_approximation_rank=2, min_compression_rate=2,
                            orthogonalization_epsilon=0, error_compressor=None)
    torch.manual_seed(0)
    tr = DataParallelTrainer(models.LeNet(), lambda p: torch.optim.SGD(p, lr=0.05), F.cross_entropy, reducer=ns,
                             device=torch.device("cpu"))
    x, y = torch.randn(8, 3, 32, 32), torch.randint(0, 10, (8,))
    for _ in range(4):
        tr.step(x, y)
    sd = tr.state_dict()
    assert sd["reducer"]["iter"] == 4 and sd["steps"] == 4
    torch.manual_seed(1)
    tr2 = DataParallelTrainer(models.LeNet(), lambda p: torch.optim.SGD(p, lr=0.05), F.cross_entropy, reducer=ns,
                              device=torch.device("cpu"))
    tr2.load_state_dict(sd)
    assert tr2.state.iter == 4 and tr2.state.ef_buffer_bytes() == tr.state.ef_buffer_bytes()
    assert torch.isfinite(tr2.step(x, y))
