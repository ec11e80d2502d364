"""Benchmark arm that runs the UNMODIFIED reference (a byte-identical copy under ``baseline/_ref``).

Everything on the measured path is the reference's own code: its model
(``examples/ImageClassification/models/wideresnet.py:44-83``), its registry
(``examples/ImageClassification/get_comm_hooks.py:9-126``), its hook
(``communication/powerSGD_hook.py:280-580``), its count sketch with its own CUDA source strings
(``communication/compressors/CountSketch.py:6-182``) and its kernel loader
(``communication/compressors/cupy_kernel.py:10-45``), on NCCL all-reduce and cuBLAS as it ships.
The training step is the reference's loop body (``examples/ImageClassification/main.py:225-231``)
under the bf16 autocast the benchmark configuration names.  What this file adds sits outside the
reference: the adapters of ``baseline/compat`` (old ``GradBucket`` method names, module aliases,
CuPy / pynvrtc call shapes on cuda-python), synthetic data and the timing protocol, which is the
one ``bench.py`` applies to the product arm.  Nothing of the product package is imported.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def _namespace(**over):
    ns = argparse.Namespace(grad_reducer="conef_powersgd", start_compression_iter=2, compression_ratio=0.1,
                            beta=0.9, sketch_size=0.1, matrix_approximation_rank=4, min_compression_rate=2,
                            orthogonalization_epsilon=0)
    for k, v in over.items():
        setattr(ns, k, v)
    return ns


def _register(example_dir, ns, ddp_net, gpu):
    """The reference's own registry of that example, unmodified (get_comm_hooks.py:9-126)."""
    import importlib

    from compat import legacy_bucket

    sys.path.insert(0, example_dir)
    for name in ("get_comm_hooks", "model", "models"):
        sys.modules.pop(name, None)
    registry = importlib.import_module("get_comm_hooks")
    registrar = legacy_bucket.HookRegistrar(ddp_net)
    state = registry.get_comm_hooks(ns, registrar, gpu)
    assert registrar.hook is not None and registrar.hook.__module__.startswith("communication."), registrar.hook
    return state


def _workload(args, device, gpu, torch):
    """Reference model + DDP + the reference's hook registration for ``args.config``.
    Returns (step(*batch) -> loss, make_batch() -> host tensors, samples per step and GPU, namespace,
    state, description)."""
    from torch.nn.parallel import DistributedDataParallel as ddp

    from compat import install

    ref = install.REF
    gen = torch.Generator().manual_seed(1234 + int(os.environ.get("RANK", 0)))
    to_dev = lambda *ts: tuple(t.to(device, non_blocking=True) for t in ts)

    if args.config == "wrn":
        example = os.path.join(ref, "examples", "ImageClassification")
        sys.path.insert(0, example)
        from models.wideresnet import Wide_ResNet             # the reference's model, unmodified
        ns = _namespace()
        batch = args.batch or 128
        net = (Wide_ResNet(16, 2, 0.3, 100) if args.small else Wide_ResNet(28, 10, 0.3, 100)).to(device)
        ddp_net = ddp(net, device_ids=[gpu], output_device=gpu)
        state = _register(example, ns, ddp_net, gpu)
        # examples/ImageClassification/main.py:190-208 with the wide-resnet defaults of its parser (:349-351)
        optimizer = torch.optim.SGD(ddp_net.parameters(), lr=0.05, momentum=0.9, weight_decay=5e-4, nesterov=True)
        criterion = torch.nn.CrossEntropyLoss()

        def make_batch():
            return torch.randn(batch, 3, 32, 32, generator=gen), torch.randint(0, 100, (batch,), generator=gen)

        def step(inputs, targets):
            # examples/ImageClassification/main.py:225-231
            inputs, targets = to_dev(inputs, targets)
            optimizer.zero_grad()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                outputs = ddp_net(inputs)
                loss = criterion(outputs, targets)
            loss.backward()
            optimizer.step()
            return loss.detach()

        desc = dict(model="WideResNet-28-10 (100 classes)" if not args.small else "WRN-16-2 (smoke)", unit="img/s",
                    dtype="bf16", seq_len=None, reducer="PowerSGD rank 4 + ConEF count sketch 10%, beta 0.9")
        return step, make_batch, batch, ns, state, desc

    if args.config == "lstm":
        # The benchmark configuration names an 8-bit quantised error store, which the reference does not
        # have; its closest reducer is the random block with classic (dense) error feedback.
        example = os.path.join(ref, "examples", "LanguageModeling")
        sys.path.insert(0, example)
        sys.modules.pop("model", None)
        from model import RNNModel                              # examples/LanguageModeling/model.py:6-62
        vocab, bptt = 33278, 35
        batch = args.batch or 20
        hid, layers = (650, 3) if not args.small else (64, 2)
        ns = _namespace(grad_reducer="ef_randomblock")
        net = RNNModel("LSTM", vocab, hid, hid, layers, 0.5, True).to(device)
        ddp_net = ddp(net, device_ids=[gpu], output_device=gpu)
        state = _register(example, ns, ddp_net, gpu)
        optimizer = torch.optim.SGD(ddp_net.parameters(), lr=1.0)
        criterion = torch.nn.NLLLoss()
        hidden_box = [None]

        def repackage(h):                                        # examples/LanguageModeling/main.py:148-154
            return h.detach() if isinstance(h, torch.Tensor) else tuple(repackage(v) for v in h)

        def make_batch():
            data = torch.randint(0, vocab, (bptt + 1, batch), generator=gen)
            return data[:-1].contiguous(), data[1:].reshape(-1).contiguous()

        def step(data, targets):
            # examples/LanguageModeling/main.py:183-199
            data, targets = to_dev(data, targets)
            if hidden_box[0] is None:
                hidden_box[0] = ddp_net.module.init_hidden(batch)
            ddp_net.zero_grad()
            hidden = repackage(hidden_box[0])
            output, hidden = ddp_net(data, hidden)
            hidden_box[0] = hidden
            loss = criterion(output, targets)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(ddp_net.parameters(), 0.25)
            optimizer.step()
            return loss.detach()

        desc = dict(model="LSTM 3x650 tied, vocab 33278", unit="tok/s", dtype="fp32", seq_len=bptt,
                    reducer="RandomBlock 10% + dense error feedback (the reference has no 8-bit error store)")
        return step, make_batch, batch * bptt, ns, state, desc

    if args.config == "transformer":
        # The configuration names low-rank compressed error feedback; the reference's hPowerSGD keeps
        # its error top-k sparsified (hPowerSGD_hook.py:90-97), which is what its registry offers.
        example = os.path.join(ref, "examples", "MachineTranslation")
        sys.path.insert(0, example)
        sys.modules.pop("model", None)
        from model import Seq2SeqTransformer                     # examples/MachineTranslation/model.py:44-88
        vocab, pad = 32000, 1
        sentences = args.batch or 37
        ns = _namespace(grad_reducer="hefsgd_powersgd", matrix_approximation_rank=8)
        if args.small:
            net = Seq2SeqTransformer(2, 2, 64, 4, vocab, vocab, 128, 0.1)
        else:
            net = Seq2SeqTransformer(6, 6, 512, 8, vocab, vocab, 2048, 0.1)
        net.tgt_tok_emb.embedding.weight = net.src_tok_emb.embedding.weight      # shared vocabulary
        net = net.to(device)
        ddp_net = ddp(net, device_ids=[gpu], output_device=gpu)
        state = _register(example, ns, ddp_net, gpu)
        optimizer = torch.optim.Adam(ddp_net.parameters(), lr=1e-4, betas=(0.9, 0.98), eps=1e-9)   # main.py:158
        criterion = torch.nn.CrossEntropyLoss(ignore_index=pad)

        def create_mask(src, tgt):
            # examples/MachineTranslation/train_n_test.py:23-41 (that module cannot be imported: it needs torchtext)
            sz = tgt.shape[0]
            mask = (torch.triu(torch.ones((sz, sz), device=device)) == 1).transpose(0, 1)
            tgt_mask = mask.float().masked_fill(mask == 0, float("-inf")).masked_fill(mask == 1, float(0.0))
            src_mask = torch.zeros((src.shape[0], src.shape[0]), device=device).type(torch.bool)
            return src_mask, tgt_mask, (src == pad).transpose(0, 1), (tgt == pad).transpose(0, 1)

        def make_batch():
            src_len = torch.randint(10, 101, (sentences,), generator=gen)
            tgt_len = torch.randint(10, 101, (sentences,), generator=gen)
            src = torch.full((101, sentences), pad, dtype=torch.long)
            tgt = torch.full((102, sentences), pad, dtype=torch.long)
            for i in range(sentences):
                src[: src_len[i], i] = torch.randint(4, vocab, (int(src_len[i]),), generator=gen)
                tgt[: tgt_len[i] + 1, i] = torch.randint(4, vocab, (int(tgt_len[i]) + 1,), generator=gen)
            return src, tgt

        def step(src, tgt):
            # examples/MachineTranslation/train_n_test.py:108-124
            src, tgt = to_dev(src, tgt)
            tgt_input = tgt[:-1, :]
            sm, tm, sp, tp = create_mask(src, tgt_input)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                logits = ddp_net(src, tgt_input, sm, tm, sp, tp, sp)
            optimizer.zero_grad()
            loss = criterion(logits.reshape(-1, logits.shape[-1]).float(), tgt[1:, :].reshape(-1))
            loss.backward()
            optimizer.step()
            return loss.detach()

        desc = dict(model="Transformer-base 6+6 (shared vocab 32000)", unit="tok/s", dtype="bf16", seq_len=101,
                    reducer="hPowerSGD rank 8 + top-k (0.4) error feedback, the reference's own error store")
        return step, make_batch, sentences * 110, ns, state, desc

    raise NotImplementedError(
        f"the reference arm covers wrn, lstm and transformer; {args.config}: the reference's BERT driver needs apex "
        "(FusedLAMB, amp) and h5py, which are not installed")


def run(args, ClockSampler, real_stdout) -> int:
    sys.path.insert(0, HERE)
    from compat import install

    try:
        install.install()
    except Exception as e:  # noqa: BLE001
        os.write(real_stdout, (json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"}) + "\n").encode())
        return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        os.write(real_stdout, (json.dumps({"impl": "reference", "unavailable":
                 "the reference's count sketch is CUDA-only (communication/compressors/CountSketch.py:108-115) "
                 "and no GPU is visible"}) + "\n").encode())
        return 0
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    gpu = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(29500 + (os.getpid() % 2000)))
    torch.cuda.set_device(gpu)
    device = torch.device("cuda", gpu)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)

    step, make_batch, per_gpu, ns, state, desc = _workload(args, device, gpu, torch)

    def sync():
        torch.cuda.synchronize(device)

    nbuf = 4
    dev_batches = [tuple(t.to(device) for t in make_batch()) for _ in range(nbuf)]
    flush = torch.empty(256 * 1024 * 1024 // 4, device=device)
    pre = ns.start_compression_iter + 7          # the same number of untimed steps as the product arm
    for i in range(pre + max(args.warmup, 0)):
        step(*dev_batches[i % nbuf])
    sync()
    assert state.iter >= ns.start_compression_iter, "the compressed path did not start"

    sampler = ClockSampler(gpu) if rank == 0 else None
    dist.barrier()
    sync()
    if sampler:
        sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    t0 = time.perf_counter()
    for i in range(args.steps):
        flush.fill_(float(i))              # evict L2 between timed steps (outside the event pair)
        starts[i].record()
        step(*dev_batches[i % nbuf])
        ends[i].record()
    sync()
    dist.barrier()
    wall = time.perf_counter() - t0
    per_step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    ms = sum(per_step_ms) / len(per_step_ms)
    t_ms = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms = float(t_ms.item())
    value = per_gpu * world / (ms / 1e3)

    e2e = None
    if not args.no_e2e:
        host = [tuple(t.pin_memory() for t in make_batch()) for _ in range(nbuf)]
        h2d = sum(t.numel() * t.element_size() for t in host[0])
        loss_host = torch.zeros(args.steps, dtype=torch.float32).pin_memory()
        for i in range(3):
            step(*host[i % nbuf])
        sync()
        dist.barrier()
        sync()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        t0 = time.perf_counter()
        for i in range(args.steps):
            loss = step(*host[i % nbuf])
            loss_host[i : i + 1].copy_(loss.float().view(1), non_blocking=True)
        ev1.record()
        sync()
        e_wall = time.perf_counter() - t0
        dist.barrier()
        e_ms = max(ev0.elapsed_time(ev1) / args.steps, e_wall * 1e3 / args.steps)
        t_e = torch.tensor([e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t_e, op=dist.ReduceOp.MAX)
        e_ms = float(t_e.item())
        e2e = {"value": per_gpu * world / (e_ms / 1e3), "unit": desc["unit"], "ms_per_step": e_ms,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4, "last_loss": float(loss_host[-1]),
               "loss_finite": bool(torch.isfinite(loss_host).all())}

    clocks = sampler.stop() if sampler else None
    if rank == 0:
        ef_bytes = 0
        for per_bucket in getattr(state, "error_dict", {}).values():
            items = per_bucket.values() if isinstance(per_bucket, dict) else \
                per_bucket if isinstance(per_bucket, (list, tuple)) else [per_bucket]
            for it in items:
                t = it.cs if hasattr(it, "cs") else it
                ef_bytes += t.numel() * t.element_size()
        out = {
            "metric": f"{desc['unit']} training throughput, {desc['model']}, {desc['reducer']}",
            "value": value, "unit": desc["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": desc["dtype"], "data": "synthetic (random-init weights, N(0,1) / uniform-id inputs)",
            "impl": "reference",
            "config": {"model": desc["model"], "global_batch": per_gpu * world, "per_gpu_batch": per_gpu,
                       "seq_len": desc.get("seq_len"), "parallelism": f"dp{world}", "reducer": ns.grad_reducer,
                       "rank": ns.matrix_approximation_rank, "sketch_size": ns.sketch_size, "beta": ns.beta,
                       "l2": "256 MB buffer written between timed steps (outside the per-step event pair)",
                       "timing": "CUDA events per step on the launching stream, mean over steps, max over ranks",
                       "comm": "nccl", "bucket_cap_mb": 25.0,
                       "code": "unmodified reference files under baseline/_ref through baseline/compat adapters"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": 0,
            "wall_s_timed_region": wall, "ef_buffer_mb": ef_bytes / 1e6,
        }
        os.write(real_stdout, (json.dumps(out) + "\n").encode())
    dist.barrier()
    dist.destroy_process_group()
    return 0
