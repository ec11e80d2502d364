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


def _workload(args, device, gpu, torch):
    """Reference model + DDP + the reference's hook registration for ``args.config``."""
    from torch.nn.parallel import DistributedDataParallel as ddp

    from compat import install, legacy_bucket

    ref = install.REF
    gen = torch.Generator().manual_seed(1234 + int(os.environ.get("RANK", 0)))
    ns = argparse.Namespace(grad_reducer="conef_powersgd", start_compression_iter=2, compression_ratio=0.1,
                            beta=0.9, sketch_size=0.1, matrix_approximation_rank=4, min_compression_rate=2,
                            orthogonalization_epsilon=0)
    if args.config != "wrn":
        raise NotImplementedError(f"the reference arm covers --config wrn, not {args.config}")
    sys.path.insert(0, os.path.join(ref, "examples", "ImageClassification"))
    import get_comm_hooks as registry                      # the reference's registry, unmodified
    from models.wideresnet import Wide_ResNet             # the reference's model, unmodified

    batch = args.batch or 128
    if args.small:
        net = Wide_ResNet(16, 2, 0.3, 100)
    else:
        net = Wide_ResNet(28, 10, 0.3, 100)
    net = net.to(device)
    ddp_net = ddp(net, device_ids=[gpu], output_device=gpu)
    registrar = legacy_bucket.HookRegistrar(ddp_net)
    state = registry.get_comm_hooks(ns, registrar, gpu)
    assert registrar.hook is not None and registrar.hook.__module__.startswith("communication."), registrar.hook
    # examples/ImageClassification/main.py:190-208 with the wide-resnet defaults of its parser (:349-351)
    optimizer = torch.optim.SGD(ddp_net.parameters(), lr=0.05, momentum=0.9, weight_decay=5e-4, nesterov=True)
    criterion = torch.nn.CrossEntropyLoss()

    def make_batch():
        return torch.randn(batch, 3, 32, 32, generator=gen), torch.randint(0, 100, (batch,), generator=gen)

    def step(inputs, targets):
        # examples/ImageClassification/main.py:225-231
        inputs, targets = inputs.to(device, non_blocking=True), targets.to(device, non_blocking=True)
        optimizer.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            outputs = ddp_net(inputs)
            loss = criterion(outputs, targets)
        loss.backward()
        optimizer.step()
        return loss.detach()

    desc = dict(model="WideResNet-28-10 (100 classes)" if not args.small else "WRN-16-2 (smoke)", unit="img/s",
                dtype="bf16", reducer="PowerSGD rank 4 + ConEF count sketch 10%, beta 0.9")
    return step, make_batch, batch, ns, state, desc


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
    pre = ns.start_compression_iter + 1
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
            items = per_bucket.values() if isinstance(per_bucket, dict) else [per_bucket]
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
                       "seq_len": None, "parallelism": f"dp{world}", "reducer": ns.grad_reducer,
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
