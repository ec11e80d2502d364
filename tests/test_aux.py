"""Auxiliary subsystems on CPU: checkpoint / resume, graceful stop, tracing, schedulers, data helpers."""
import os
import signal

import numpy as np
import pytest
import torch

import conef_b200 as cb
from conef_b200 import data, optim, utils
from conef_b200.ops import reference as ref

from helpers import FakeBucket, free_port

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
    # the GPU-only options are inert on a CPU run: no graphs are captured, cuDNN's switch is left alone
    before = torch.backends.cudnn.benchmark
    tr3 = DataParallelTrainer(models.LeNet(), lambda p: torch.optim.SGD(p, lr=0.05), F.cross_entropy, reducer=None,
                              device=torch.device("cpu"), cudnn_autotune=True,
                              graph_modules=lambda m: [m], graph_sample_inputs=(x,))
    assert tr3.graphed_modules == 0 and (torch.cuda.is_available() or torch.backends.cudnn.benchmark == before)
    assert torch.isfinite(tr3.step(x, y))
    torch.backends.cudnn.benchmark = before


def _toy_corpus(tmp_path):
    words = ["the", "cat", "dog", "sat", "ran", "on", "mat", "fast", "slow", "blue", "red", "house", "tree", "##s", "##ing"]
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + words
    vf = tmp_path / "vocab.txt"
    vf.write_text("\n".join(vocab) + "\n")
    import random
    rng = random.Random(0)
    lines = []
    for d in range(12):
        for s in range(rng.randint(3, 7)):
            lines.append(" ".join(rng.choice(words[:13]) for _ in range(rng.randint(4, 12))))
        lines.append("")
    cf = tmp_path / "corpus.txt"
    cf.write_text("\n".join(lines))
    return vf, cf


def test_pretraining_instances_shards_and_prefetch(tmp_path):
    """Documents -> sentence-pair / masked-LM instances -> .npz shards -> dataset, following the
    recipe of the reference's create_pretraining_data.py."""
    from conef_b200 import data as D
    vf, cf = _toy_corpus(tmp_path)
    tok = D.BertTokenizer(str(vf))
    docs = D.read_documents([str(cf)], tok)
    assert len(docs) == 12 and all(len(d) >= 3 for d in docs)
    inst = D.create_training_instances(docs, list(tok.vocab.keys()), max_seq_length=32, dupe_factor=3,
                                       max_predictions_per_seq=5, seed=1)
    assert len(inst) >= 12 * 3
    n_random = 0
    for it in inst:
        assert it.tokens[0] == "[CLS]" and it.tokens[-1] == "[SEP]" and it.tokens.count("[SEP]") == 2
        assert len(it.tokens) <= 32 and len(it.tokens) == len(it.segment_ids)
        first_sep = it.tokens.index("[SEP]")
        assert set(it.segment_ids[: first_sep + 1]) == {0} and set(it.segment_ids[first_sep + 1 :]) == {1}
        assert 1 <= len(it.masked_lm_positions) <= 5 and len(it.masked_lm_positions) == len(it.masked_lm_labels)
        assert all(it.tokens[p] not in ("[CLS]", "[SEP]") or it.tokens[p] == "[MASK]" for p in it.masked_lm_positions)
        assert 0 not in it.masked_lm_positions
        n_random += it.is_random_next
    assert 0.2 < n_random / len(inst) < 0.8
    # shards
    half = len(inst) // 2
    for k, part in enumerate((inst[:half], inst[half:])):
        D.write_shard(str(tmp_path / f"part_{k}.npz"), D.instances_to_arrays(part, tok, 32, 5))
    files = D.shard_files(str(tmp_path), rank=0, world=2, epoch=0) + D.shard_files(str(tmp_path), rank=1, world=2, epoch=0)
    assert sorted(files) == sorted(str(tmp_path / f"part_{k}.npz") for k in range(2))
    assert len(D.shard_files(str(tmp_path), rank=3, world=4)) == 1            # fewer files than ranks: wrap
    total = 0
    pre = D.ShardPrefetcher(sorted(files), 5)
    for shard in pre:
        assert isinstance(shard, D.PretrainingShard)
        ids, seg, mask, labels, nsp = shard[0]
        assert ids.shape == (32,) and seg.shape == (32,) and mask.shape == (32,) and labels.shape == (32,)
        assert int(mask.sum()) >= 5 and nsp in (0, 1)
        assert 1 <= int((labels >= 0).sum()) <= 5 and bool((labels[mask == 0] == -1).all())
        assert int(ids[0]) == tok.vocab["[CLS]"]
        total += len(shard)
    pre.close()
    assert total == len(inst)
    # the first instance survives the round trip
    first = D.PretrainingShard(str(tmp_path / "part_0.npz"))[0]
    want_ids = tok.convert_tokens_to_ids(inst[0].tokens)
    assert first[0][: len(want_ids)].tolist() == want_ids
    for p, lab in zip(inst[0].masked_lm_positions, tok.convert_tokens_to_ids(inst[0].masked_lm_labels)):
        assert int(first[3][p]) == lab


def test_bert_driver_trains_from_shard_files(tmp_path):
    """create_pretraining_data.py -> run_pretraining.py --input_dir, end to end on CPU."""
    import subprocess, sys, json
    vf, cf = _toy_corpus(tmp_path)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()), RANK="0", WORLD_SIZE="1",
               CUDA_VISIBLE_DEVICES="")
    shards = tmp_path / "shards"
    subprocess.run([sys.executable, os.path.join(root, "examples/bert_pretraining/create_pretraining_data.py"),
                    "--input_file", str(cf), "--vocab_file", str(vf), "--output_prefix", str(shards / "part"),
                    "--shards", "2", "--max_seq_length", "32", "--max_predictions_per_seq", "5", "--dupe_factor", "2"],
                   check=True, env=env, timeout=300)
    assert len(list(shards.glob("*.npz"))) == 2
    out = tmp_path / "run"
    subprocess.run([sys.executable, os.path.join(root, "examples/bert_pretraining/run_pretraining.py"),
                    "--bert_model", "tiny", "--input_dir", str(shards), "--output_dir", str(out),
                    "--max_seq_length", "32", "--max_predictions_per_seq", "5", "--train_batch_size", "4",
                    "--max_steps", "6", "--grad_reducer", "conef_powersgd", "--matrix_approximation_rank", "2"],
                   check=True, env=env, timeout=600)
    lines = [json.loads(l) for l in (out / "log.jsonl").read_text().splitlines()]
    assert any(l.get("step") == "summary" for l in lines)


def test_glue_processors_and_features(tmp_path):
    from conef_b200.data import glue
    vf, _ = _toy_corpus(tmp_path)
    tok = data.BertTokenizer(str(vf))
    d = tmp_path / "mrpc"
    d.mkdir()
    (d / "train.tsv").write_text("Quality\t#1 ID\t#2 ID\t#1 String\t#2 String\n"
                                 "1\t11\t12\tthe cat sat\tthe dog ran fast\n0\t13\t14\tblue house\tred tree\n")
    (d / "dev.tsv").write_text("Quality\t#1 ID\t#2 ID\t#1 String\t#2 String\n1\t1\t2\tcat\tdog\n")
    proc = glue.PROCESSORS["mrpc"]()
    train = proc.get_train_examples(str(d))
    assert [(e.text_a, e.text_b, e.label) for e in train] == [("the cat sat", "the dog ran fast", "1"),
                                                              ("blue house", "red tree", "0")]
    assert len(proc.get_dev_examples(str(d))) == 1 and proc.get_labels() == ["0", "1"]
    feats = glue.convert_examples_to_features(train, proc.get_labels(), 12, tok)
    f = feats[0]
    assert len(f.input_ids) == len(f.input_mask) == len(f.segment_ids) == 12 and f.label_id == 1
    assert f.input_ids[0] == tok.vocab["[CLS]"] and sum(f.input_mask) == 3 + 3 + 4
    assert f.segment_ids[:5] == [0] * 5 and f.segment_ids[5:10] == [1] * 5 and f.segment_ids[10:] == [0, 0]
    # truncation keeps the pair within the budget; single sentences get one separator
    short = glue.convert_examples_to_features(train, proc.get_labels(), 8, tok)[0]
    assert sum(short.input_mask) == 8 and short.input_ids.count(tok.vocab["[SEP]"]) == 2
    c = tmp_path / "cola"
    c.mkdir()
    (c / "train.tsv").write_text("gj04\t1\t\tthe cat sat on the mat\n")
    ex = glue.DataProcessor("CoLA").get_train_examples(str(c))[0]
    assert (ex.text_a, ex.text_b, ex.label) == ("the cat sat on the mat", None, "1")
    one = glue.convert_examples_to_features([ex], ["0", "1"], 16, tok)[0]
    assert one.input_ids.count(tok.vocab["[SEP]"]) == 1 and set(one.segment_ids) == {0}
    with pytest.raises(KeyError):
        glue.DataProcessor("nope")


def test_extract_features_script(tmp_path):
    import json, subprocess, sys
    vf, _ = _toy_corpus(tmp_path)
    (tmp_path / "in.txt").write_text("the cat sat ||| the dog ran\n\nblue house\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.run([sys.executable, os.path.join(root, "examples/bert_pretraining/extract_features.py"),
                    "--input_file", str(tmp_path / "in.txt"), "--output_file", str(tmp_path / "out.jsonl"),
                    "--vocab_file", str(vf), "--bert_model", "tiny", "--layers=-1,-2", "--max_seq_length", "16",
                    "--no_cuda"], check=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    lines = [json.loads(l) for l in (tmp_path / "out.jsonl").read_text().splitlines()]
    assert [l["linex_index"] for l in lines] == [0, 1]
    first = lines[0]["features"]
    assert [f["token"] for f in first] == ["[CLS]", "the", "cat", "sat", "[SEP]", "the", "dog", "ran", "[SEP]"]
    assert [l["index"] for l in first[0]["layers"]] == [-1, -2] and len(first[0]["layers"][0]["values"]) == 128


def test_question_answering_span_selection(tmp_path):
    import importlib.util, json, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "examples/bert_pretraining/inference.py")
    spec = importlib.util.spec_from_file_location("qa_inference", path)
    qa = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(qa)
    vf, _ = _toy_corpus(tmp_path)
    tok = data.BertTokenizer(str(vf))
    ids, mask, seg, tokens, t2w, words = qa.build_features("the cat", "the dog sat on the mat fast", tok, 16, 4)
    assert tokens == ["[CLS]", "the", "cat", "[SEP]", "the", "dog", "sat", "on", "the", "mat", "fast", "[SEP]"]
    assert len(ids) == len(mask) == len(seg) == 16 and sum(mask) == 12
    assert t2w == [-1, -1, -1, -1, 0, 1, 2, 3, 4, 5, 6, -1]
    start = [0.0] * 12
    end = [0.0] * 12
    start[6], end[9] = 5.0, 4.0          # "sat on the mat"
    start[1] = 9.0                       # inside the question: never an answer
    best = qa.best_spans(start, end, t2w, words, n_best_size=3, max_answer_length=10)
    assert best[0]["text"] == "sat on the mat" and best[0]["start_logit"] == 5.0
    assert qa.best_spans(start, end, t2w, words, n_best_size=3, max_answer_length=2)[0]["text"] != "sat on the mat"
    start[0], end[0] = 20.0, 20.0        # strong [CLS]: the empty answer wins when allowed
    assert qa.best_spans(start, end, t2w, words, 3, 10, with_negative=True)[0]["text"] == ""
    out = subprocess.run([sys.executable, path, "--vocab_file", str(vf), "--bert_model", "tiny", "--no_cuda",
                          "--question", "the cat", "--context", "the dog sat on the mat", "--max_seq_length", "16",
                          "--n_best_size", "3"], check=True, capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    res = json.loads(out.stdout.strip().splitlines()[-1])
    assert res["question"] == "the cat" and isinstance(res["answers"][0]["text"], str)


def test_bert_driver_phase_two_starts_from_phase_one_weights(tmp_path):
    """--init_checkpoint: a new run (fresh optimizer and reducer state) from the weights of another."""
    import json, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "examples/bert_pretraining/run_pretraining.py")

    def run(out, *extra):
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()), RANK="0", WORLD_SIZE="1",
                   CUDA_VISIBLE_DEVICES="")
        subprocess.run([sys.executable, script, "--bert_model", "tiny", "--output_dir", str(out),
                        "--train_batch_size", "4", "--max_steps", "4", "--shard_size", "32",
                        "--grad_reducer", "ef_powersgd", "--matrix_approximation_rank", "2", *extra],
                       check=True, env=env, timeout=600)
    run(tmp_path / "p1", "--max_seq_length", "32", "--max_predictions_per_seq", "5")
    run(tmp_path / "p2", "--max_seq_length", "64", "--max_predictions_per_seq", "10",
        "--init_checkpoint", str(tmp_path / "p1"), "--resume_from_checkpoint")
    a = torch.load(utils.latest_checkpoint(str(tmp_path / "p1")), map_location="cpu", weights_only=False)
    b = torch.load(utils.latest_checkpoint(str(tmp_path / "p2")), map_location="cpu", weights_only=False)
    assert a["step"] == 4 and b["step"] == 4          # phase 2 counted its own steps
    moved = sum(float((a["model"][k].float() - b["model"][k].float()).abs().sum()) for k in a["model"])
    assert moved > 0
    with pytest.raises(subprocess.CalledProcessError):
        run(tmp_path / "p3", "--init_checkpoint", str(tmp_path / "nothing_here"))


def test_bert_driver_single_process_and_post_accumulation_modes(tmp_path):
    """--local_rank -1 (no process group; DataParallel when several GPUs are visible) and
    --allreduce_post_accumulation[_fp16] (no DDP: one flat all-reduce per optimizer step, two gloo ranks)."""
    import json, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "examples/bert_pretraining/run_pretraining.py")
    common = ["--bert_model", "tiny", "--train_batch_size", "4", "--max_steps", "3", "--shard_size", "32",
              "--max_seq_length", "32", "--max_predictions_per_seq", "5"]

    def summary(out):
        lines = [json.loads(l) for l in open(os.path.join(out, "log.jsonl"))]
        return [l for l in lines if l.get("step") == "summary"][-1]

    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    subprocess.run([sys.executable, script, *common, "--output_dir", str(tmp_path / "single"), "--local_rank", "-1",
                    "--grad_reducer", "allreduce"], check=True, env=env, timeout=600)
    s1 = summary(str(tmp_path / "single"))
    assert s1["mode"] == "single device" and np.isfinite(s1["final_loss"])

    port = str(free_port())
    procs = []
    for r in range(2):
        e = dict(env, MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK="0")
        procs.append(subprocess.Popen([sys.executable, script, *common, "--output_dir", str(tmp_path / "post"),
                                       "--gradient_accumulation_steps", "2", "--allreduce_post_accumulation",
                                       "--allreduce_post_accumulation_fp16", "--local_rank", "0"], env=e))
    assert [p.wait(timeout=600) for p in procs] == [0, 0]
    s2 = summary(str(tmp_path / "post"))
    assert s2["mode"] == "post-accumulation all-reduce" and np.isfinite(s2["final_loss"])
    assert s2["allreduce_mb_per_step"] > 0 and s2["ef_buffer_mb"] == 0.0


def test_post_accumulation_allreduce_averages_over_ranks():
    from conef_b200.parallel.accumulate import PostAccumulationAllReduce, broadcast_parameters
    from helpers import run_ranks

    run_ranks(_post_accumulation_worker, world=2, args=(), backend="gloo")


def _post_accumulation_worker(rank, world):
    import torch.distributed as dist
    from conef_b200.parallel.accumulate import PostAccumulationAllReduce, broadcast_parameters

    torch.manual_seed(100 + rank)
    net = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 2))
    broadcast_parameters(net)
    flat = torch.cat([p.detach().reshape(-1) for p in net.parameters()])
    both = [torch.zeros_like(flat) for _ in range(world)]
    dist.all_gather(both, flat)
    assert torch.equal(both[0], both[1])                     # every rank starts from rank 0's weights
    for dtype, tol in ((torch.float32, 1e-6), (torch.float16, 2e-3)):
        net.zero_grad()
        for micro in range(2):                                # two micro-batches accumulate locally
            net(torch.randn(3, 6)).pow(2).sum().backward()
        local = torch.cat([p.grad.reshape(-1) for p in net.parameters()]).clone()
        gathered = [torch.zeros_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        red = PostAccumulationAllReduce(net.parameters(), wire_dtype=dtype, accumulation_steps=2,
                                        predivide_accumulation=True)
        assert red.allreduce()
        got = torch.cat([p.grad.reshape(-1) for p in net.parameters()])
        torch.testing.assert_close(got, sum(gathered) / (world * 2), rtol=tol, atol=tol * 10)
        assert red.bytes_on_wire == local.numel() * (4 if dtype == torch.float32 else 2)


def test_parallel_text_and_translation_driver(tmp_path):
    import subprocess, sys
    src = ["ein mann geht .", "eine frau liest ein buch .", "der hund rennt schnell !", "", "ein kind spielt ."] * 8
    tgt = ["a man walks .", "a woman reads a book .", "the dog runs fast !", "", "a child plays ."] * 8
    (tmp_path / "train.de").write_text("\n".join(src) + "\n")
    (tmp_path / "train.en").write_text("\n".join(tgt) + "\n")
    ds = data.ParallelText(str(tmp_path / "train.de"), str(tmp_path / "train.en"))
    assert len(ds) == 32                                           # empty lines dropped on both sides
    assert list(ds.src_vocab)[:4] == ["<unk>", "<pad>", "<bos>", "<eos>"] and ds.src_vocab["."] == 4
    s0, t0 = ds[0]
    assert ds.decode(t0) == "a man walks ." and ds.decode(s0, "src") == "ein mann geht ."
    batch_src, batch_tgt = data.collate_translation([ds[0], ds[1]])
    assert batch_src.shape == (8, 2) and int(batch_src[0, 0]) == 2 and int(batch_src[5, 0]) == 3
    assert int(batch_src[7, 0]) == 1                               # padded behind EOS
    other = data.ParallelText(str(tmp_path / "train.de"), str(tmp_path / "train.en"), ds.src_vocab, {"<unk>": 0})
    assert set(other[0][1].tolist()) == {0}                        # unknown words map to <unk>
    (tmp_path / "short.en").write_text("one line\n")
    with pytest.raises(ValueError):
        data.ParallelText(str(tmp_path / "train.de"), str(tmp_path / "short.en"))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()), RANK="0", WORLD_SIZE="1",
               CUDA_VISIBLE_DEVICES="")
    subprocess.run([sys.executable, os.path.join(root, "examples/machine_translation/main.py"),
                    "--train_src", str(tmp_path / "train.de"), "--train_tgt", str(tmp_path / "train.en"),
                    "--batch_size", "8", "--emb_size", "32", "--nhead", "2", "--ffn_hid_dim", "64",
                    "--num_encoder_layers", "1", "--num_decoder_layers", "1", "--start_compression_iter", "2",
                    "--matrix_approximation_rank", "2", "--grad_reducer", "ef_powersgd"],
                   check=True, env=env, timeout=600)


def test_image_driver_evaluates_and_writes_the_results_folder(tmp_path):
    """Test accuracy per epoch on rank 0, learning-rate decay epochs, results pickles and a README that
    --resume appends to (reference examples/ImageClassification/main.py:23-66,238-257,287-306)."""
    import subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "examples/image_classification/main.py")

    def run(*extra):
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()), RANK="0", WORLD_SIZE="1",
                   CUDA_VISIBLE_DEVICES="")
        subprocess.run([sys.executable, script, "--model", "lenet", "--epochs", "2", "--steps_per_epoch", "3",
                        "--test_steps", "2", "--batch_size", "8", "--grad_reducer", "ef_powersgd",
                        "--start_compression_iter", "2", "--results", str(tmp_path), "--name", "run",
                        "--lr_decay_at_epoch1", "1", *extra], check=True, env=env, timeout=600)
    run()
    folder = tmp_path / "run"
    acc = utils.load_obj(str(folder / "test_accuracies"))
    assert len(acc) == 2 and all(0.0 <= a <= 100.0 for a in acc)
    assert len(utils.load_obj(str(folder / "train_losses"))) == 2 and len(utils.load_obj(str(folder / "time_per_epoch"))) == 2
    hist = utils.load_obj(str(folder / "results"))["history"]
    assert hist[1]["lr"] == pytest.approx(hist[0]["lr"] / 10)
    readme = (folder / "README.md").read_text()
    assert "grad_reducer: ef_powersgd\\" in readme and "best_acc:" in readme
    run("--resume", "1")
    assert (folder / "README.md").read_text().count("grad_reducer: ef_powersgd") == 2


def test_corpus_formatting_segmentation_and_sharding(tmp_path):
    """wikiextractor / books formatting -> rule-based sentences -> balanced shards -> .npz instances
    (reference data/WikicorpusTextFormatting.py, BookscorpusTextFormatting.py, TextSharding.py, bertPrep.py)."""
    import subprocess, sys
    from conef_b200.data import corpus_prep as cp

    seg = cp.RuleSegmenter()
    assert seg.segment_string('Dr. Smith went to Washington. He arrived at 3 p.m. on Monday! "Was it late?" No.') == \
        ["Dr. Smith went to Washington.", "He arrived at 3 p.m. on Monday!", '"Was it late?"', "No."]
    assert seg.segment_string("One sentence only") == ["One sentence only"]

    wd = tmp_path / "data"
    wiki = wd / "download" / "wikicorpus_en" / "AA"
    wiki.mkdir(parents=True)
    docs = []
    for k in range(12):
        body = " ".join(f"Article {k} sentence {j} is here." for j in range(1 + (k * 7) % 9))
        docs.append(f'<doc id="{k}" url="u" title="T{k}">\nT{k}\n\n{body}\n</doc>\n')
    (wiki / "wiki_00").write_text("".join(docs[:6]))
    (wiki / "wiki_01").write_text("".join(docs[6:]))
    books = wd / "download" / "bookscorpus"
    books.mkdir(parents=True)
    for k in range(5):
        (books / f"book{k}.txt").write_text("\n".join(f"Book {k} line {j} ends here." for j in range(3 + k)) + "\n\n")
    out = wd / "fmt"
    out.mkdir()
    assert cp.format_wikicorpus(str(wd / "download" / "wikicorpus_en"), str(out / "wiki.txt")) == 12
    assert cp.format_bookscorpus(str(books), str(out / "books.txt")) == 5
    lines = (out / "wiki.txt").read_text().splitlines()
    assert lines[0].startswith("Article 0 sentence 0") and "T0" not in lines[0]       # the title line is dropped

    sh = cp.Sharding([str(out / "wiki.txt"), str(out / "books.txt")], str(tmp_path / "shards" / "corpus"), 3, 2, 0.25)
    sh.load_articles()
    sh.segment_articles_into_sentences()
    sh.distribute_articles_over_shards()
    files = sh.write_shards_to_disk()
    assert [os.path.basename(f) for f in files] == ["corpus_training_0.txt", "corpus_training_1.txt",
                                                     "corpus_training_2.txt", "corpus_test_0.txt", "corpus_test_1.txt"]
    placed = sorted(a for shard in list(sh.output_training_files.values()) + list(sh.output_test_files.values())
                    for a in shard)
    assert placed == list(range(17))                                 # every article exactly once
    train = [sh.sentences_per_shard(s) for s in sh.output_training_files.values()]
    test = [sh.sentences_per_shard(s) for s in sh.output_test_files.values()]
    total = sum(train) + sum(test)
    assert max(train) - min(train) <= 9 and abs(sum(test) / total - 0.25) < 0.12
    text = open(files[0]).read()
    assert text.endswith("\n\n") and "\n\n\n" not in text            # sentence per line, blank line between articles
    with pytest.raises(ValueError):
        cp.Sharding([str(out / "books.txt")], str(tmp_path / "x"), 4, 4, 0.1).distribute_articles_over_shards()

    # the command-line pipeline end to end on the books
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "examples/bert_pretraining/prep_corpus.py")
    vocab = tmp_path / "vocab.txt"
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "book", "line", "ends", "here", ".", "0", "1", "2", "3", "4",
             "5", "6", "7"]
    vocab.write_text("\n".join(words) + "\n")
    common = [sys.executable, script, "--dataset", "bookscorpus", "--working_dir", str(wd), "--n_training_shards", "2",
              "--n_test_shards", "1", "--fraction_test_set", "0.2"]
    subprocess.run(common + ["--action", "text_formatting"], check=True, timeout=300)
    subprocess.run(common + ["--action", "sharding"], check=True, timeout=300)
    subprocess.run(common + ["--action", "create_pretraining_files", "--vocab_file", str(vocab), "--max_seq_length", "32",
                             "--max_predictions_per_seq", "5"], check=True, timeout=300)
    import glob
    npz = glob.glob(str(wd / "npz" / "**" / "*.npz"), recursive=True)
    assert len(npz) == 3
    shard = data.pretraining.load_shard(npz[0])
    assert shard["input_ids"].shape[1] == 32
    assert subprocess.run(common + ["--action", "download"], capture_output=True).returncode != 0


def test_hardware_presets_print_their_settings():
    """configs/pretrain_config.sh: presets per machine shape (reference scripts/configs/pretrain_config.sh)."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "examples/bert_pretraining/configs/pretrain_config.sh")
    out = subprocess.run(["bash", script, "b200_8gpu_bf16_conef"], capture_output=True, text=True, check=True).stdout
    got = dict(line.split("=", 1) for line in out.split())
    assert got["GPUS"] == "8" and got["REDUCER"] == "conef_powersgd" and got["RANK_R"] == "8"
    assert int(got["GPUS"]) * int(got["BATCH1"]) * int(got["ACCUM1"]) == 8192      # the LAMB recipe's global batch
    assert int(got["GPUS"]) * int(got["BATCH2"]) * int(got["ACCUM2"]) == 4096
    one = dict(l.split("=", 1) for l in subprocess.run(["bash", script, "b200_1gpu_bf16_conef"], capture_output=True,
                                                       text=True, check=True).stdout.split())
    assert int(one["GPUS"]) * int(one["BATCH1"]) * int(one["ACCUM1"]) == 8192
    post = subprocess.run(["bash", script, "b200_8gpu_bf16_post_accumulation"], capture_output=True, text=True,
                          check=True).stdout
    assert "POST_ACCUMULATION_FP16=1" in post and "REDUCER=allreduce" in post


def test_cluster_and_container_launch_files_parse():
    """The SLURM batch file and the container scripts (reference: run.sub, Dockerfile, scripts/docker/*) cannot
    run here (no scheduler, no container runtime): their shell syntax is checked and the batch file is
    expanded with a fake `srun` to see the command a node would run."""
    import subprocess
    import tempfile
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ex = os.path.join(root, "examples/bert_pretraining")
    for f in ("run.sub", "docker/build.sh", "docker/launch.sh"):
        subprocess.run(["bash", "-n", os.path.join(ex, f)], check=True)
    assert "conef_b200.ops.build" in open(os.path.join(ex, "Dockerfile")).read()
    with tempfile.TemporaryDirectory() as d:
        for name, body in (("srun", 'echo "SRUN $@"'), ("scontrol", "echo node-a; echo node-b")):
            path = os.path.join(d, name)
            with open(path, "w") as fh:
                fh.write("#!/bin/bash\n" + body + "\n")
            os.chmod(path, 0o755)
        env = dict(os.environ, PATH=d + os.pathsep + os.environ["PATH"], SLURM_JOB_NODELIST="node-[a-b]",
                   SLURM_JOB_NUM_NODES="2", SLURM_SUBMIT_DIR=root, PHASE="2", REDUCER="ef_powersgd", OUT=os.path.join(d, "out"))
        out = subprocess.run(["bash", os.path.join(ex, "run.sub")], capture_output=True, text=True, check=True, env=env).stdout
    assert "--nnodes 2" in out and "--master_addr node-a" in out and "--max_seq_length 512" in out
    assert "--grad_reducer ef_powersgd" in out and "--init_checkpoint results/bert/phase1" in out


def test_model_repository_export_and_in_process_client(tmp_path):
    """Export a tiny QA model as a served-model repository, check ``config.pbtxt`` and the exported-against-eager
    errors, then answer questions and a SQuAD file through the in-process back end of the client."""
    import importlib.util, json, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, rel))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    exp = load("deploy_export", "examples/bert_pretraining/deploy/export.py")
    cli = load("deploy_client", "examples/bert_pretraining/deploy/client.py")
    vf, _ = _toy_corpus(tmp_path)
    tok = data.BertTokenizer(str(vf))
    repo = tmp_path / "repo"
    rep = exp.main(["--repository", str(repo), "--model_name", "qa", "--bert_model", "tiny", "--tiny_vocab",
                    str(max(len(tok.vocab), 8)), "--max_seq_length", "32", "--batch_size", "3", "--no_cuda",
                    "--dynamic_batching_delay_us", "50", "--preferred_batch_sizes", "2", "--tolerance", "1e-5"])
    assert rep["check"]["max_linf"] <= 1e-5 and rep["check"]["tensors_compared"] == 6
    assert rep["input_dims"] == [[-1]] * 3 and rep["output_dims"] == [[-1]] * 2      # the sequence axis is dynamic
    text = (repo / "qa" / "config.pbtxt").read_text()
    assert 'platform: "pytorch_libtorch"' in text and "max_batch_size: 3" in text and "KIND_CPU" in text
    assert text.count("TYPE_INT64") == 3 and text.count("TYPE_FP32") == 2 and "preferred_batch_size: [2]" in text
    assert (repo / "qa" / "1" / "model.pt").exists()
    cfg = cli.read_config(str(repo / "qa" / "config.pbtxt"))
    assert cfg == {"max_batch_size": 3, "inputs": ["input__0", "input__1", "input__2"],
                   "outputs": ["output__0", "output__1"]}

    backend = cli.LocalBackend(str(repo), "qa", device="cpu")
    pairs = [("the cat", "the dog sat on the mat fast")] * 5 + [("the dog", "the cat sat")] * 2
    spans = cli.answer_batch(backend, tok, pairs, max_seq_length=24, max_query_length=4, n_best_size=3)
    assert len(spans) == 7 and spans[0] == spans[4] and all(isinstance(s[0]["text"], str) for s in spans)
    # seven requests went through in chunks of max_batch_size = 3 and equal the one-by-one answers
    single = cli.answer_batch(backend, tok, pairs[5:6], max_seq_length=24, max_query_length=4, n_best_size=3)
    assert single[0] == spans[5]

    squad = {"data": [{"paragraphs": [{"context": "the dog sat on the mat",
                                       "qas": [{"id": "q1", "question": "the cat"}, {"id": "q2", "question": "the mat"}]}]}]}
    sf = tmp_path / "dev.json"
    sf.write_text(json.dumps(squad))
    out = tmp_path / "pred.json"
    preds = cli.main(["--local_repository", str(repo), "--model_name", "qa", "--vocab_file", str(vf), "--device", "cpu",
                      "--squad_file", str(sf), "--output_file", str(out), "--max_seq_length", "24", "--batch_size", "2"])
    assert set(preds) == {"q1", "q2"} and json.loads(out.read_text()) == preds
    perf = cli.main(["--local_repository", str(repo), "--model_name", "qa", "--device", "cpu", "--perf",
                     "--batch_size", "4", "--max_seq_length", "16", "--perf_iters", "2", "--perf_vocab", "8"])
    assert perf["seq_per_s"] > 0 and perf["batch_size"] == 4
    import subprocess
    csv_path = tmp_path / "perf.csv"
    subprocess.run(["bash", os.path.join(root, "examples/bert_pretraining/deploy/run_perf.sh"), "1", "3"], check=True,
                   capture_output=True, timeout=300,
                   env=dict(os.environ, REPOSITORY=str(repo), MODEL_NAME="qa", SEQ_LENGTH="16", ITERS="2", PERF_VOCAB="8",
                            DEVICE="cpu", OUT=str(csv_path), CUDA_VISIBLE_DEVICES=""))
    table = csv_path.read_text().splitlines()
    assert table[0] == "batch_size,seq_length,seq_per_s,ms_per_request" and [r.split(",")[0] for r in table[1:]] == ["1", "3"]
    with pytest.raises(RuntimeError, match="tritonclient"):
        cli.TritonBackend("127.0.0.1:8000", "qa")
    gold = {"data": [{"paragraphs": [{"context": "c", "qas": [
        {"id": "a", "answers": [{"text": "The Mat."}, {"text": "a rug"}]},
        {"id": "b", "answers": [{"text": "on the red mat"}]}, {"id": "c", "answers": [{"text": "dog"}]}]}]}]}
    gf = tmp_path / "gold.json"
    gf.write_text(json.dumps(gold))
    sc = cli.squad_scores({"a": "mat", "b": "the mat", "c": "cat"}, str(gf))
    # a: exact after normalisation; b: one of three gold words, precision 1 and recall 1/3, F1 = 0.5; c: nothing shared
    assert sc["questions"] == 3 and abs(sc["exact_match"] - 100 / 3) < 1e-9 and abs(sc["f1"] - 50.0) < 1e-9
    assert exp.dynamic_dims([(torch.zeros(2, 5, 7),), (torch.zeros(3, 5, 9),)]) == [[5, -1]]


def test_serving_scripts_parse_and_dry_run():
    """The server launch needs a container runtime: its command line is printed instead (DRY_RUN=1); the wait
    script gives up after its limit when nothing listens; the export script chains exporter and client."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d = os.path.join(root, "examples/bert_pretraining/deploy")
    for f in ("launch_server.sh", "wait_for_server.sh", "export_model.sh"):
        subprocess.run(["bash", "-n", os.path.join(d, f)], check=True)
    env = dict(os.environ, DRY_RUN="1", REPOSITORY="/models/repo", GPUS="0,1")
    out = subprocess.run(["bash", os.path.join(d, "launch_server.sh")], capture_output=True, text=True, check=True, env=env).stdout
    assert "--gpus device=0,1" in out and "-v /models/repo:/models:ro" in out and "tritonserver --model-repository=/models" in out
    out = subprocess.run(["bash", os.path.join(d, "export_model.sh"), "ck.pt", "4", "fp16", "ts-trace", "128"],
                         capture_output=True, text=True, check=True,
                         env=dict(env, VOCAB_FILE="v.txt", SQUAD_FILE="dev.json", BERT_MODEL="base")).stdout.splitlines()
    assert len(out) == 3 and "export.py" in out[0] and "--fp16" in out[0] and "--init_checkpoint ck.pt" in out[0]
    assert "--squad_file dev.json --evaluate" in out[1] and "--perf" in out[2]
    r = subprocess.run(["bash", os.path.join(d, "wait_for_server.sh"), "127.0.0.1:%d" % free_port(), "1"],
                       capture_output=True, text=True)
    assert r.returncode == 1 and "did not become ready" in r.stderr


def test_glue_fine_tuning_driver_trains_evaluates_and_reloads(tmp_path):
    """The sentence-pair fine-tuning driver on a toy task (label 1 when the first sentence has a cat): the loss
    falls, the dev metrics are written, and an evaluation-only run from the saved weights repeats them; a
    pre-training checkpoint contributes its encoder and leaves the classifier fresh."""
    import importlib.util, json, random
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("run_glue", os.path.join(root, "examples/bert_pretraining/run_glue.py"))
    rg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rg)
    vf, _ = _toy_corpus(tmp_path)
    rng = random.Random(1)
    words = ["dog", "sat", "ran", "on", "mat", "fast", "slow", "blue", "red", "house", "tree"]

    def rows(n):
        out = ["Quality\t#1 ID\t#2 ID\t#1 String\t#2 String"]
        for i in range(n):
            a = [rng.choice(words) for _ in range(rng.randint(2, 5))]
            lab = i % 2
            if lab:
                a[rng.randrange(len(a))] = "cat"
            b = [rng.choice(words) for _ in range(rng.randint(2, 5))]
            out.append(f"{lab}\t{i}\t{i}\t{' '.join(a)}\t{' '.join(b)}")
        return "\n".join(out) + "\n"
    d = tmp_path / "mrpc"
    d.mkdir()
    (d / "train.tsv").write_text(rows(96))
    (d / "dev.tsv").write_text(rows(32))
    out = tmp_path / "out"
    common = ["--task_name", "mrpc", "--data_dir", str(d), "--vocab_file", str(vf), "--bert_model", "tiny", "--no_cuda",
              "--max_seq_length", "16", "--output_dir", str(out)]
    res = rg.main(common + ["--do_train", "--do_eval", "--train_batch_size", "16", "--gradient_accumulation_steps", "2",
                            "--learning_rate", "5e-4", "--num_train_epochs", "10"])
    assert res["train_steps"] == 60 and res["train_loss_last"] < 0.5 * res["train_loss_first"]
    assert res["eval_examples"] == 32 and res["eval_accuracy"] >= 0.9 and 0.0 <= res["eval_f1"] <= 1.0
    assert json.loads((out / "eval_results.json").read_text())["eval_accuracy"] == res["eval_accuracy"]
    again = rg.main(common + ["--do_eval", "--init_checkpoint", str(out / "pytorch_model.pt")])
    assert again["eval_accuracy"] == res["eval_accuracy"] and again["tensors_not_in_checkpoint"] == 0
    assert abs(again["eval_loss"] - res["eval_loss"]) < 1e-6
    # a pre-training checkpoint: encoder tensors are taken, the two classifier tensors stay fresh
    from conef_b200 import models
    sd = torch.load(out / "pytorch_model.pt")["model"]
    pre = {k: v for k, v in sd.items() if not k.startswith("classifier.")}
    torch.save({"model": pre}, tmp_path / "pre.pt")
    third = rg.main(common + ["--do_eval", "--init_checkpoint", str(tmp_path / "pre.pt")])
    assert third["tensors_not_in_checkpoint"] == 2
    m = rg.classification_metrics("cola", [1, 1, 0, 0], [1, 0, 0, 0])
    assert abs(m["mcc"] - (1 * 2 - 1 * 0) / (2 * 1 * 3 * 2) ** 0.5) < 1e-12 and m["accuracy"] == 0.75
    assert rg.classification_metrics("mrpc", [1, 1, 0], [1, 0, 1])["f1"] == 0.5
    assert "f1" not in rg.classification_metrics("sst-2", [1], [1])


def test_glue_launcher_and_presets_dry_run(tmp_path):
    """Task x machine presets split the global batch into per-GPU batch and accumulation; the launcher turns them
    into the driver's command line (printed under DRY_RUN=1) and runs evaluation alone on one GPU."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ex = os.path.join(root, "examples/bert_pretraining")
    for f in ("run_glue.sh", "configs/glue_config.sh"):
        subprocess.run(["bash", "-n", os.path.join(ex, f)], check=True)
    script = (f"source {ex}/configs/glue_config.sh && glue_sst2 && b200_1gpu_fp32 && glue_show && "
              f"glue_mrpc && b200_8gpu_bf16 && glue_show && DRY_RUN=1 OUT={tmp_path}/o bash {ex}/run_glue.sh && "
              f"MODE=eval DRY_RUN=1 OUT={tmp_path}/o CHECKPOINT=ck.pt bash {ex}/run_glue.sh")
    out = subprocess.run(["bash", "-c", script], capture_output=True, text=True, check=True).stdout.splitlines()
    assert "TASK=sst-2 GPUS=1 BATCH=256 ACCUM=4" in out[0] and "PRECISION=fp32" in out[0]
    assert "TASK=mrpc GPUS=8 BATCH=16 ACCUM=1" in out[1]
    assert "--nproc-per-node 8" in out[2] and "--task_name mrpc" in out[2] and "--do_train --do_eval --bf16" in out[2]
    assert "torch.distributed.run" not in out[3] and "--do_train" not in out[3] and "--init_checkpoint ck.pt" in out[3]


def _toy_squad(path, n, rng, with_impossible=False):
    filler = ["dog", "sat", "ran", "on", "mat", "fast", "slow", "house", "tree", "the"]
    paragraphs = []
    for i in range(n):
        words = [rng.choice(filler) for _ in range(rng.randint(6, 14))]
        impossible = with_impossible and i % 4 == 3
        qa = {"id": f"q{i}", "question": "the cat"}
        if not impossible:
            pos = rng.randrange(len(words))
            words[pos] = rng.choice(["blue", "red"])
        context = " ".join(words)
        if impossible:
            qa.update({"answers": [], "is_impossible": True})
        else:
            start = len(" ".join(words[:pos])) + (1 if pos else 0)
            qa["answers"] = [{"text": words[pos], "answer_start": start}]
            assert context[start:start + len(words[pos])] == words[pos]
        paragraphs.append({"context": context, "qas": [qa]})
    path.write_text(__import__("json").dumps({"data": [{"title": "toy", "paragraphs": paragraphs}]}))


def test_squad_features_windows_and_answers(tmp_path):
    from conef_b200.data import squad
    vf, _ = _toy_corpus(tmp_path)
    tok = data.BertTokenizer(str(vf))
    words, c2w = squad.split_context("the  cat sat\ton the mat")
    assert words == ["the", "cat", "sat", "on", "the", "mat"] and c2w[:5] == [0, 0, 0, 0, 0] and c2w[5] == 1
    ctx = "the dog sat on the blue mat fast the cats ran on the red house slow"
    doc = {"data": [{"paragraphs": [{"context": ctx, "qas": [
        {"id": "a", "question": "the cat", "answers": [{"text": "blue mat", "answer_start": ctx.index("blue mat")}]},
        {"id": "b", "question": "the dog", "answers": [{"text": "cat", "answer_start": ctx.index("cats")}]},
        {"id": "c", "question": "the tree", "answers": [], "is_impossible": True},
        {"id": "bad", "question": "x", "answers": [{"text": "zebra", "answer_start": 3}]}]}]}]}
    f = tmp_path / "s.json"
    f.write_text(__import__("json").dumps(doc))
    train = squad.read_squad_examples(str(f), True, with_negative=True)
    assert [e.qas_id for e in train] == ["a", "b", "c"]              # the mis-annotated answer is dropped
    assert (train[0].start_word, train[0].end_word) == (5, 6) and train[2].is_impossible
    assert len(squad.read_squad_examples(str(f), False)) == 4
    # 17 pieces ("cats" is two), 2 question pieces: max_seq_length 14 leaves room for 9, stride 4 -> windows at 0, 4, 8
    feats = squad.convert_examples_to_features(train, tok, max_seq_length=14, doc_stride=4, max_query_length=4, is_training=True)
    fa = [x for x in feats if x.example_index == 0]
    assert [x.window for x in fa] == [0, 1, 2] and all(len(x.input_ids) == 14 for x in fa)
    assert fa[0].tokens[:4] == ["[CLS]", "the", "cat", "[SEP]"] and fa[0].tokens[4:13] == ctx.split()[:9]
    assert (fa[0].start_position, fa[0].end_position) == (4 + 5, 4 + 6)           # "blue mat" inside window 0
    assert (fa[1].start_position, fa[1].end_position) == (4 + 1, 4 + 2)           # window 1 starts at piece 4
    assert (fa[2].start_position, fa[2].end_position) == (0, 0)                   # not in window 2: [CLS]
    # every context piece has exactly one best window, and it is the one where it sits deepest
    owners = {}
    for x in fa:
        for t, (w, best) in enumerate(zip(x.token_to_word, x.max_context)):
            if best:
                piece = (x.window * 4) + t - 4
                assert piece not in owners
                owners[piece] = x.window
    assert sorted(owners) == list(range(17)) and owners[0] == 0 and owners[16] == 2 and owners[8] == 1
    fb = [x for x in feats if x.example_index == 1]
    s, e = fb[1].start_position, fb[1].end_position
    assert fb[1].tokens[s:e + 1] == ["cat"]                                       # the answer is one piece of "cats"
    assert all((x.start_position, x.end_position) == (0, 0) for x in feats if x.example_index == 2)
    # answers: logits that point at "red house" in the last window; the same span seen from a worse window is ignored
    ex = squad.read_squad_examples(str(f), False, with_negative=True)[:1]
    pf = squad.convert_examples_to_features(ex, tok, 14, 4, 4)
    sl = [[0.0] * 14 for _ in pf]
    el = [[0.0] * 14 for _ in pf]
    t_red = pf[2].tokens.index("red")
    sl[2][t_red], el[2][t_red + 1] = 5.0, 5.0
    ans, ranked = squad.best_answers(ex, pf, sl, el, n_best_size=5, max_answer_length=4)
    assert ans == {"a": "red house"} and ranked["a"][0]["score"] == 10.0
    sl[0][0] = el[0][0] = sl[1][0] = el[1][0] = sl[2][0] = el[2][0] = 9.0          # strong [CLS] in every window
    assert squad.best_answers(ex, pf, sl, el, 5, 4, with_negative=True)[0] == {"a": ""}
    assert squad.best_answers(ex, pf, sl, el, 5, 4, with_negative=True, null_score_diff_threshold=20.0)[0] == {"a": "red house"}
    sc = squad.squad_scores({"a": "Blue mat.", "b": "cats", "c": "", "bad": "zebra"}, str(f))
    assert sc["questions"] == 4 and sc["exact_match"] == 75.0


def test_squad_fine_tuning_driver_learns_a_toy_task(tmp_path):
    """The answer is the one colour word of the context: after fine-tuning, exact match on held-out contexts is
    high; predictions, n-best lists and the checkpoint are written; the checkpoint feeds the export tool."""
    import importlib.util, json, random
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("run_squad", os.path.join(root, "examples/bert_pretraining/run_squad.py"))
    rs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rs)
    vf, _ = _toy_corpus(tmp_path)
    rng = random.Random(3)
    _toy_squad(tmp_path / "train.json", 96, rng)
    _toy_squad(tmp_path / "dev.json", 24, rng)
    out = tmp_path / "out"
    res = rs.main(["--do_train", "--do_predict", "--do_eval", "--train_file", str(tmp_path / "train.json"),
                   "--predict_file", str(tmp_path / "dev.json"), "--vocab_file", str(vf), "--bert_model", "tiny", "--no_cuda",
                   "--max_seq_length", "24", "--doc_stride", "8", "--max_query_length", "4", "--train_batch_size", "16",
                   "--learning_rate", "1e-3", "--num_train_epochs", "15", "--output_dir", str(out), "--n_best_size", "5"])
    assert res["train_windows"] == 96 and res["train_steps"] == 90 and res["train_loss_last"] < 0.3 * res["train_loss_first"]
    assert res["questions"] == 24 and res["exact_match"] >= 85.0 and res["f1"] >= res["exact_match"]
    preds = json.loads((out / "predictions.json").read_text())
    assert len(preds) == 24 and sum(p in ("blue", "red") for p in preds.values()) >= 20
    assert len(json.loads((out / "nbest_predictions.json").read_text())["q0"]) >= 1
    again = rs.main(["--do_predict", "--do_eval", "--predict_file", str(tmp_path / "dev.json"), "--vocab_file", str(vf),
                     "--bert_model", "tiny", "--no_cuda", "--max_seq_length", "24", "--doc_stride", "8", "--max_query_length", "4",
                     "--init_checkpoint", str(out / "pytorch_model.pt"), "--output_dir", str(tmp_path / "out2"), "--n_best_size", "5"])
    assert again["exact_match"] == res["exact_match"] and again["tensors_not_in_checkpoint"] == 0


def test_squad_launcher_and_presets_dry_run(tmp_path):
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ex = os.path.join(root, "examples/bert_pretraining")
    for f in ("run_squad.sh", "configs/squad_config.sh"):
        subprocess.run(["bash", "-n", os.path.join(ex, f)], check=True)
    script = (f"source {ex}/configs/squad_config.sh && squad_b200_8gpu_bf16_conef && "
              f"DRY_RUN=1 OUT={tmp_path}/o SQUAD_DIR=sq bash {ex}/run_squad.sh && "
              f"MODE=eval VERSION=2.0 DRY_RUN=1 OUT={tmp_path}/o SQUAD_DIR=sq CHECKPOINT=ck.pt bash {ex}/run_squad.sh")
    out = subprocess.run(["bash", "-c", script], capture_output=True, text=True, check=True).stdout.splitlines()
    assert "--nproc-per-node 8" in out[0] and "--train_file sq/train-v1.1.json" in out[0] and "--grad_reducer conef_powersgd" in out[0]
    assert "--do_predict --do_eval --predict_file sq/dev-v1.1.json" in out[0] and out[0].endswith("--bf16")
    assert "torch.distributed.run" not in out[1] and "--do_train" not in out[1] and "--version_2_with_negative" in out[1]
    assert "--predict_file sq/dev-v2.0.json" in out[1] and "--init_checkpoint ck.pt" in out[1]


def test_swag_multiple_choice_driver(tmp_path):
    """Four endings, the right one holds a cat: the shared encoder with a one-logit head learns to pick it."""
    import csv, importlib.util, random, subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ex = os.path.join(root, "examples/bert_pretraining")
    spec = importlib.util.spec_from_file_location("run_swag", os.path.join(ex, "run_swag.py"))
    sw = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sw)
    vf, _ = _toy_corpus(tmp_path)
    rng = random.Random(5)
    filler = ["dog", "sat", "ran", "on", "mat", "fast", "slow", "house", "tree", "blue", "red"]
    d = tmp_path / "swag"
    d.mkdir()

    def write(name, n):
        with open(d / name, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["", "video-id", "fold-ind", "startphrase", "sent1", "sent2", "gold-source",
                        "ending0", "ending1", "ending2", "ending3", "label"])
            for i in range(n):
                sent = lambda k: " ".join(rng.choice(filler) for _ in range(k))
                label = rng.randrange(4)
                ends = [sent(3) for _ in range(4)]
                ends[label] = "cat " + sent(2)
                w.writerow([i, "v", i, "", sent(4), "the", "gold", *ends, label])
    write("train.csv", 64)
    write("val.csv", 24)
    rows = sw.read_swag(str(d / "val.csv"))
    assert len(rows) == 24 and len(rows[0][2]) == 4 and rows[0][1] == "the" and "cat" in rows[0][2][rows[0][3]]
    tok = data.BertTokenizer(str(vf))
    ids, seg, mask, lab = sw.choice_features(rows[:2], tok, 16)
    assert len(ids) == 2 and len(ids[0]) == 4 and len(ids[0][0]) == 16 and lab == [rows[0][3], rows[1][3]]
    assert ids[0][0][:6] == ids[0][1][:6] and ids[0][rows[0][3]].count(tok.vocab["cat"]) == 1     # shared context
    out = tmp_path / "out"
    common = ["--data_dir", str(d), "--vocab_file", str(vf), "--bert_model", "tiny", "--no_cuda", "--max_seq_length", "16",
              "--output_dir", str(out)]
    res = sw.main(common + ["--do_train", "--do_eval", "--train_batch_size", "8", "--learning_rate", "1e-3",
                            "--num_train_epochs", "8"])
    assert res["num_choices"] == 4 and res["train_steps"] == 64 and res["train_loss_last"] < 0.5 * res["train_loss_first"]
    assert res["eval_examples"] == 24 and res["eval_accuracy"] >= 0.85
    again = sw.main(common + ["--do_eval", "--init_checkpoint", str(out / "pytorch_model.pt")])
    assert again["eval_accuracy"] == res["eval_accuracy"] and again["tensors_not_in_checkpoint"] == 0
    subprocess.run(["bash", "-n", os.path.join(ex, "run_swag.sh")], check=True)
    line = subprocess.run(["bash", os.path.join(ex, "run_swag.sh")], capture_output=True, text=True, check=True,
                          env=dict(os.environ, DRY_RUN="1", OUT=str(tmp_path / "o"), MODE="eval", CHECKPOINT="ck.pt")).stdout
    assert "run_swag.py" in line and "--do_eval" in line and "--do_train" not in line and "torch.distributed.run" not in line


def test_fine_tuning_on_two_gloo_ranks_with_a_compression_hook(tmp_path):
    """The shared fine-tuning loop under DDP on two CPU ranks with PowerSGD + count-sketch error feedback:
    both ranks run the same number of steps, rank 0 writes the results, the task is learnt."""
    import json, random, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    vf, _ = _toy_corpus(tmp_path)
    rng = random.Random(1)
    words = ["dog", "sat", "ran", "on", "mat", "fast", "slow", "blue", "red", "house", "tree"]

    def rows(n):
        out = ["Quality\t#1 ID\t#2 ID\t#1 String\t#2 String"]
        for i in range(n):
            a = [rng.choice(words) for _ in range(rng.randint(2, 5))]
            if i % 2:
                a[rng.randrange(len(a))] = "cat"
            out.append(f"{i % 2}\t{i}\t{i}\t{' '.join(a)}\t{' '.join(rng.choice(words) for _ in range(3))}")
        return "\n".join(out) + "\n"
    d = tmp_path / "mrpc"
    d.mkdir()
    (d / "train.tsv").write_text(rows(96))
    (d / "dev.tsv").write_text(rows(32))
    out = tmp_path / "out"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(root, "examples/bert_pretraining/run_glue.py"),
           "--task_name", "mrpc", "--data_dir", str(d), "--vocab_file", str(vf), "--bert_model", "tiny", "--no_cuda",
           "--max_seq_length", "16", "--output_dir", str(out), "--do_train", "--do_eval", "--train_batch_size", "8",
           "--learning_rate", "5e-4", "--num_train_epochs", "10", "--grad_reducer", "conef_powersgd",
           "--matrix_approximation_rank", "2"]
    subprocess.run(cmd, check=True, capture_output=True, text=True, timeout=600, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    res = json.loads((out / "eval_results.json").read_text())
    assert res["world_size"] == 2 and res["grad_reducer"] == "conef_powersgd" and res["train_steps"] == 60
    assert res["train_loss_last"] < 0.3 * res["train_loss_first"] and res["eval_accuracy"] >= 0.9


def test_cluster_presets_keep_the_recipes_global_batch_and_drive_the_batch_file(tmp_path):
    import importlib.util, subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ex = os.path.join(root, "examples/bert_pretraining")
    spec = importlib.util.spec_from_file_location("cluster_preset", os.path.join(ex, "cluster_preset.py"))
    cp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cp)
    presets = cp.load()
    assert len(presets) >= 10 and not any(k.startswith(".") for k in presets)
    for name, v in presets.items():
        assert cp.global_batch(v) == (8192 if v["PHASE"] == "1" else 4096), name
        assert name.startswith(f"bert--B200_{v['NNODES']}x{v['GPUS']}x{v['BATCH']}x{v['ACCUM']}")
    assert presets["bert--B200_4x8x64x4_allreduce"]["REDUCER"] == "allreduce"
    assert cp.main(["nope"]) == 2
    for name, body in (("srun", 'echo "SRUN $@"'), ("scontrol", "echo node-a; echo node-b")):
        path = tmp_path / name
        path.write_text("#!/bin/bash\n" + body + "\n")
        path.chmod(0o755)
    script = (f'eval "$({sys_executable()} {ex}/cluster_preset.py bert--B200_4x8x16x8_phase2)" && '
              f'OUT={tmp_path}/out bash {ex}/run.sub')
    env = dict(os.environ, PATH=str(tmp_path) + os.pathsep + os.environ["PATH"], SLURM_JOB_NODELIST="node-[a-d]",
               SLURM_JOB_NUM_NODES="4", SLURM_SUBMIT_DIR=root)
    out = subprocess.run(["bash", "-c", script], capture_output=True, text=True, check=True, env=env).stdout
    assert "--max_seq_length 512" in out and "--train_batch_size 128 --gradient_accumulation_steps 8" in out
    assert "--learning_rate 4e-3" in out and "--max_steps 1563" in out and "--grad_reducer conef_powersgd" in out


def sys_executable():
    import sys
    return sys.executable


def test_dataset_creation_script_runs_both_phases_from_raw_books(tmp_path):
    """create_datasets.sh chains formatting, sharding and instance creation for sequence lengths 128 and 512."""
    import glob, subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "examples/bert_pretraining/create_datasets.sh")
    subprocess.run(["bash", "-n", script], check=True)
    dry = subprocess.run(["bash", script, "wiki_books"], capture_output=True, text=True, check=True,
                         env=dict(os.environ, DRY_RUN="1")).stdout.splitlines()
    assert len(dry) == 5 and "--dataset bookscorpus" in dry[0] and "--dataset wikicorpus_en" in dry[1]
    assert "--action sharding --dataset books_wiki_en_corpus" in dry[2]
    assert "--max_seq_length 128 --max_predictions_per_seq 20" in dry[3] and "--max_seq_length 512" in dry[4]
    assert subprocess.run(["bash", script, "nope"], capture_output=True).returncode == 2
    wd = tmp_path / "data"
    books = wd / "download" / "bookscorpus"
    books.mkdir(parents=True)
    for k in range(6):
        (books / f"book{k}.txt").write_text("\n".join(f"Book {k} line {j} ends here." for j in range(4 + k)) + "\n\n")
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("\n".join(["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "book", "line", "ends", "here", "."]
                               + [str(i) for i in range(10)]) + "\n")
    env = dict(os.environ, WORKING_DIR=str(wd), VOCAB=str(vocab), SHARDS_TRAIN="2", SHARDS_TEST="1", TEST_FRACTION="0.2",
               CUDA_VISIBLE_DEVICES="")
    subprocess.run(["bash", script, "books_only"], check=True, timeout=600, env=env, capture_output=True)
    npz = glob.glob(str(wd / "npz" / "**" / "*.npz"), recursive=True)
    lengths = sorted({data.pretraining.load_shard(f)["input_ids"].shape[1] for f in npz})
    assert len(npz) == 6 and lengths == [128, 512]


def test_squad_driver_with_unanswerable_questions(tmp_path):
    """Version-2 style data: a quarter of the contexts hold no colour word and must get the empty answer."""
    import importlib.util, json, random
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("run_squad_v2", os.path.join(root, "examples/bert_pretraining/run_squad.py"))
    rs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rs)
    vf, _ = _toy_corpus(tmp_path)
    rng = random.Random(7)
    _toy_squad(tmp_path / "train.json", 128, rng, with_impossible=True)
    _toy_squad(tmp_path / "dev.json", 32, rng, with_impossible=True)
    out = tmp_path / "out"
    res = rs.main(["--do_train", "--do_predict", "--do_eval", "--version_2_with_negative",
                   "--train_file", str(tmp_path / "train.json"), "--predict_file", str(tmp_path / "dev.json"),
                   "--vocab_file", str(vf), "--bert_model", "tiny", "--no_cuda", "--max_seq_length", "24", "--doc_stride", "8",
                   "--max_query_length", "4", "--train_batch_size", "16", "--learning_rate", "1e-3", "--num_train_epochs", "15",
                   "--output_dir", str(out), "--n_best_size", "5"])
    preds = json.loads((out / "predictions.json").read_text())
    gold = json.loads((tmp_path / "dev.json").read_text())["data"][0]["paragraphs"]
    empty_gold = {p["qas"][0]["id"] for p in gold if p["qas"][0].get("is_impossible")}
    assert len(empty_gold) == 8
    hits = sum(preds[q] == "" for q in empty_gold)
    false_empty = sum(preds[q] == "" for q in preds if q not in empty_gold)
    assert res["exact_match"] >= 80.0 and hits >= 6 and false_empty <= 4
    nbest = json.loads((out / "nbest_predictions.json").read_text())
    assert all(any(c["text"] == "" for c in nbest[q]) for q in preds)         # the empty answer always competes


def test_squad_prediction_is_shared_by_the_ranks(tmp_path):
    """Two gloo ranks train, then each scores half of the windows and rank 0 assembles the answers: the file equals
    what one process predicts from the saved weights."""
    import json, random, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "examples/bert_pretraining/run_squad.py")
    vf, _ = _toy_corpus(tmp_path)
    rng = random.Random(9)
    _toy_squad(tmp_path / "train.json", 64, rng)
    _toy_squad(tmp_path / "dev.json", 21, rng)
    common = ["--predict_file", str(tmp_path / "dev.json"), "--vocab_file", str(vf), "--bert_model", "tiny", "--no_cuda",
              "--max_seq_length", "16", "--doc_stride", "4", "--max_query_length", "4", "--n_best_size", "5", "--predict_batch_size", "4"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                    "127.0.0.1", "--master-port", str(free_port()), script, "--do_train", "--do_predict", "--do_eval",
                    "--train_file", str(tmp_path / "train.json"), "--train_batch_size", "8", "--learning_rate", "1e-3",
                    "--num_train_epochs", "4", "--output_dir", str(tmp_path / "two")] + common,
                   check=True, capture_output=True, text=True, timeout=600, env=env)
    two = json.loads((tmp_path / "two" / "results.json").read_text())
    assert two["world_size"] == 2 and two["predict_ranks"] == 2 and two["predict_windows"] > two["predict_questions"] == 21
    subprocess.run([sys.executable, script, "--do_predict", "--do_eval", "--init_checkpoint", str(tmp_path / "two" / "pytorch_model.pt"),
                    "--output_dir", str(tmp_path / "one")] + common, check=True, capture_output=True, text=True, timeout=600, env=env)
    one = json.loads((tmp_path / "one" / "results.json").read_text())
    assert one["predict_ranks"] == 1 and one["exact_match"] == two["exact_match"]
    assert json.loads((tmp_path / "one" / "predictions.json").read_text()) == json.loads((tmp_path / "two" / "predictions.json").read_text())


def test_example_drivers_on_two_gloo_ranks(tmp_path):
    """Image, language-modelling and translation drivers under torchrun with two CPU ranks and a compression hook
    each: they finish, and rank 0 reports a finite loss."""
    import json, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = ["ein mann geht .", "eine frau liest ein buch .", "der hund rennt schnell !", "ein kind spielt ."] * 8
    tgt = ["a man walks .", "a woman reads a book .", "the dog runs fast !", "a child plays ."] * 8
    (tmp_path / "train.de").write_text("\n".join(src) + "\n")
    (tmp_path / "train.en").write_text("\n".join(tgt) + "\n")
    runs = {
        "image_classification": ["--model", "lenet", "--epochs", "2", "--steps_per_epoch", "3", "--test_steps", "2",
                                 "--batch_size", "8", "--grad_reducer", "conef_powersgd", "--start_compression_iter", "2",
                                 "--results", str(tmp_path), "--name", "run"],
        "language_modeling": ["--model", "LSTM", "--tied", "--emsize", "32", "--nhid", "32", "--nlayers", "1", "--epochs", "1",
                              "--batch_size", "8", "--bptt", "8", "--vocab", "50", "--tokens", "2000",
                              "--grad_reducer", "conef_randomblock", "--start_compression_iter", "2"],
        "machine_translation": ["--train_src", str(tmp_path / "train.de"), "--train_tgt", str(tmp_path / "train.en"),
                                "--batch_size", "8", "--emb_size", "32", "--nhead", "2", "--ffn_hid_dim", "64",
                                "--num_encoder_layers", "1", "--num_decoder_layers", "1", "--start_compression_iter", "2",
                                "--matrix_approximation_rank", "2", "--grad_reducer", "hefsgd_powersgd"],
    }
    for name, args in runs.items():
        out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                              "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
                              os.path.join(root, "examples", name, "main.py"), *args],
                             check=True, capture_output=True, text=True, timeout=600,
                             env=dict(os.environ, CUDA_VISIBLE_DEVICES="")).stdout
        last = json.loads([l for l in out.splitlines() if l.startswith("{")][-1])
        loss = last.get("loss", last.get("train_loss"))
        assert loss is not None and loss == loss and abs(loss) < 1e6, (name, last)


def test_bert_pretraining_driver_on_two_gloo_ranks(tmp_path):
    """Synthetic shards, PowerSGD + count-sketch error feedback, accumulation over two micro-batches, two ranks."""
    import json, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
                          os.path.join(root, "examples/bert_pretraining/run_pretraining.py"), "--bert_model", "tiny",
                          "--max_steps", "6", "--train_batch_size", "4", "--max_seq_length", "32", "--max_predictions_per_seq", "5",
                          "--output_dir", str(tmp_path / "out"), "--shard_size", "64", "--grad_reducer", "conef_powersgd",
                          "--matrix_approximation_rank", "2", "--gradient_accumulation_steps", "2"],
                         check=True, capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, CUDA_VISIBLE_DEVICES="")).stdout
    summary = json.loads([l for l in out.splitlines() if '"summary"' in l][-1])
    assert summary["mode"] == "ddp+hook" and summary["final_loss"] == summary["final_loss"] and summary["ef_buffer_mb"] > 0
