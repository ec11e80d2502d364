#!/usr/bin/env python
"""Benchmark driver: training throughput with compressed gradient all-reduce.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Flagship configuration (``--config wrn``): WideResNet-28-10, 100 classes, bf16
autocast, batch 128 per GPU of synthetic 3x32x32 N(0,1) images, SGD momentum
0.9, PowerSGD rank-4 hook with ConEF count-sketch error compression
(sketch = 10 % of the gradient).  Rank 0 prints ONE JSON line.

``value`` is images per second over all GPUs, timed on the device (CUDA events
per step, L2 flushed between steps, max over ranks).  ``e2e`` repeats the
measurement through :class:`conef_b200.DataParallelTrainer` with the inputs
of every step copied from pinned host memory and the loss of every step copied
back to the host.  ``--impl restated`` runs the same model with the hooks
executed as PyTorch ops + NCCL all-reduce in the reference's op order (with
its one device synchronisation per bucket); ``--impl allreduce`` is plain
uncompressed DDP.  ``--impl reference`` runs the unmodified reference (a
byte-identical copy under ``baseline/_ref``: its model, registry, hook, sketch
kernels, NCCL + cuBLAS) through the adapters of ``baseline/compat`` with the same
timing protocol; the product package is not imported on that path.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
if REPO not in sys.path:
    sys.path.insert(0, REPO)



def run_reference(args) -> int:
    """``--impl reference``: the unmodified reference (``baseline/_ref``) through ``baseline/reference_arm.py``.

    The product package must not be importable on this path: the repository root also holds a
    ``communication`` alias package that would shadow the reference's directory of that name."""
    import importlib.util

    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or os.getcwd()) != REPO]
    try:
        spec = importlib.util.spec_from_file_location("reference_arm", os.path.join(REPO, "baseline", "reference_arm.py"))
        arm = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(arm)
        rc = arm.run(args, ClockSampler, real_stdout)
        assert "conef_b200" not in sys.modules, "the reference arm must not load the product package"
        return rc
    except Exception as e:  # noqa: BLE001
        import traceback
        traceback.print_exc()
        if int(os.environ.get("RANK", "0")) == 0:
            line = {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e).splitlines()[0] if str(e) else ''}"[:300]}
            os.write(real_stdout, (json.dumps(line) + "\n").encode())
        return 0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "restated", "allreduce"])
    ap.add_argument("--config", default="wrn", choices=["wrn", "resnet20", "lstm", "transformer", "bert"])
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch (default: the config's)")
    ap.add_argument("--error-compressor", default=None,
                    help="replace the configuration's error store (e.g. topk, the reference's own hPowerSGD "
                         "store, for --config transformer); the headline configurations leave it unset")
    ap.add_argument("--no-graph", action="store_true", help="do not capture the model's blocks as CUDA graphs")
    ap.add_argument("--bucket-cap-mb", type=float, default=None, help="DDP bucket size (default: the trainer's)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--small", action="store_true", help="shrunken model, for smoke tests only (not a valid number)")
    return ap.parse_args()


# --------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.1):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nvml = None

    def _loop(self):
        n = self.nvml
        names = {
            getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    n.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------
def build_workload(args, device, world):
    """Returns (model, optimizer_factory, loss_fn, make_batch(on_host) -> (inputs, target),
    samples_per_step_per_gpu, reducer namespace, autocast dtype, description dict)."""
    import torch
    import torch.nn.functional as F

    from conef_b200 import models
    from conef_b200.optim import FusedSGD

    ns = argparse.Namespace(grad_reducer="conef_powersgd", start_compression_iter=2, compression_ratio=0.1,
                            beta=0.9, sketch_size=0.1, matrix_approximation_rank=4, min_compression_rate=2,
                            orthogonalization_epsilon=0, error_compressor=None)
    gen = torch.Generator().manual_seed(1234 + (int(os.environ.get("RANK", 0))))
    if args.config == "wrn":
        batch = args.batch or 128
        model = models.WideResNet(16, 2, 0.3, 100) if args.small else models.WideResNet28_10(100)
        opt = lambda p: FusedSGD(p, lr=0.05, momentum=0.9, nesterov=True, weight_decay=5e-4)
        loss_fn = F.cross_entropy

        def make_batch():
            return (torch.randn(batch, 3, 32, 32, generator=gen),), torch.randint(0, 100, (batch,), generator=gen)
        desc = dict(model="WideResNet-28-10 (100 classes)" if not args.small else "WRN-16-2 (smoke)",
                    unit="img/s", dtype="bf16", seq_len=None, reducer="PowerSGD rank 4 + ConEF count sketch 10%, beta 0.9")
        tkw = dict(channels_last=True, cudnn_autotune=os.environ.get("CONEF_CUDNN_AUTOTUNE", "1") == "1")
        if not args.no_graph:      # forward and backward of the twelve blocks as CUDA graphs: the step is host-bound otherwise
            tkw.update(graph_modules=lambda m: list(m.blocks), graph_sample_inputs=make_batch()[0])
        return model, opt, loss_fn, make_batch, batch, ns, torch.bfloat16, desc, tkw
    if args.config == "resnet20":
        batch = args.batch or 32
        ns.matrix_approximation_rank = 2
        ns.error_compressor = "count_sketch3"
        ns.hash_seed = 7
        model = models.ResNet20(10)
        opt = lambda p: FusedSGD(p, lr=0.1, momentum=0.9)

        def make_batch():
            return (torch.randn(batch, 3, 32, 32, generator=gen),), torch.randint(0, 10, (batch,), generator=gen)
        desc = dict(model="ResNet-20", unit="img/s", dtype="fp32", seq_len=None,
                    reducer="PowerSGD rank 2 + EF + 3-row count sketch 10%")
        return model, opt, F.cross_entropy, make_batch, batch, ns, None, desc, {}
    from conef_b200 import bench_configs
    return bench_configs.build(args, device, world, ns, gen)


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)

    # Keep stdout to the one JSON line: libraries (NCCL's version banner, for one) write there,
    # so file descriptor 1 points at stderr while the benchmark runs and the line goes to the real stdout.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist

    if args.impl == "restated":
        os.environ["CONEF_BACKEND"] = "torch"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    if world != args.gpus and rank == 0:
        sys.stderr.write(f"note: WORLD_SIZE={world} but --gpus {args.gpus}; using WORLD_SIZE\n")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(29500 + (os.getpid() % 2000)))
    if use_cuda:
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world)

    from conef_b200 import DataParallelTrainer
    from conef_b200.ops import native

    model, opt_factory, loss_fn, make_batch, per_gpu, ns, ac_dtype, desc, tkw = build_workload(args, device, world)
    if args.impl == "allreduce":
        ns.grad_reducer = "allreduce"
    if args.error_compressor:
        ns.error_compressor = args.error_compressor
        desc["reducer"] += f" [error store replaced by {args.error_compressor}]"
    if not use_cuda:
        ac_dtype = None
        tkw = {k: v for k, v in tkw.items() if k != "channels_last"}
    if args.bucket_cap_mb:
        tkw["bucket_cap_mb"] = args.bucket_cap_mb
    trainer = DataParallelTrainer(model, opt_factory, loss_fn, reducer=ns, device=device,
                                  autocast_dtype=ac_dtype, **tkw)
    if args.impl == "restated" and trainer.state is not None:
        # the reference blocks the host once per bucket (powerSGD_hook.py:552-553)
        from conef_b200.parallel import hooks as _h
        _h.SYNC_EVERY_BUCKET = True

    def sync():
        if use_cuda:
            torch.cuda.synchronize(device)

    # ---- device-resident inputs for the device-timed arm -------------------
    nbuf = 4
    dev_batches = []
    for _ in range(nbuf):
        inp, tgt = make_batch()
        dev_batches.append((tuple(t.to(device) for t in inp),
                            tuple(t.to(device) for t in tgt) if isinstance(tgt, tuple) else tgt.to(device)))
    flush = torch.empty(256 * 1024 * 1024 // 4, device=device) if use_cuda else None

    # untimed: get past the warm-up all-reduce iterations of the hook and past the executor's
    # bring-up (two direct runs per buffer slot, then one graph capture per slot), then W warm-up steps
    pre = ns.start_compression_iter + 7 if ns.grad_reducer != "allreduce" else 0
    for i in range(pre + max(args.warmup, 0)):
        trainer.step(*dev_batches[i % nbuf])
    sync()
    trainer.check()

    def timed_steps(n):
        """Mean device time per step over n steps (CUDA events per step on the launching stream,
        L2 flushed before each, barrier + synchronise on both sides), max over ranks; wall seconds."""
        dist.barrier()
        sync()
        if use_cuda:
            starts = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
            ends = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        t0 = time.perf_counter()
        per = []
        for i in range(n):
            if use_cuda:
                flush.fill_(float(i))          # evict L2 between timed steps (outside the event pair)
                starts[i].record()
                trainer.step(*dev_batches[i % nbuf])
                ends[i].record()
            else:
                t = time.perf_counter()
                trainer.step(*dev_batches[i % nbuf])
                per.append((time.perf_counter() - t) * 1e3)
        sync()
        dist.barrier()
        wall_s = time.perf_counter() - t0
        if use_cuda:
            per = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        t_ms = torch.tensor([sum(per) / len(per)], device=device, dtype=torch.float64)
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
        return float(t_ms.item()), wall_s

    sampler = ClockSampler(local_rank) if use_cuda and rank == 0 else None
    dist.barrier()
    sync()
    native.reset_launch_count()
    if sampler:
        sampler.start()
    ms, wall = timed_steps(args.steps)
    launches = native.reset_launch_count()
    trainer.check()
    value = per_gpu * world / (ms / 1e3)

    # ---- end-to-end arm: pinned host inputs every step, loss read back every step ----
    e2e = None
    if not args.no_e2e:
        host = []
        for _ in range(nbuf):
            inp, tgt = make_batch()
            pin = (lambda t: t.pin_memory()) if use_cuda else (lambda t: t)
            host.append((tuple(pin(t) for t in inp), tuple(pin(t) for t in tgt) if isinstance(tgt, tuple) else pin(tgt)))
        h2d = sum(t.numel() * t.element_size() for t in host[0][0]) + \
            sum(t.numel() * t.element_size() for t in (host[0][1] if isinstance(host[0][1], tuple) else (host[0][1],)))
        loss_host = torch.zeros(args.steps, dtype=torch.float32)
        if use_cuda:
            loss_host = loss_host.pin_memory()
        for i in range(3):
            trainer.step(*host[i % nbuf])
        sync()
        dist.barrier()
        sync()
        if use_cuda:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        t0 = time.perf_counter()
        for i in range(args.steps):
            loss = trainer.step(*host[i % nbuf])
            loss_host[i : i + 1].copy_(loss.float().view(1), non_blocking=True)
        if use_cuda:
            ev1.record()
        sync()
        e_wall = time.perf_counter() - t0
        dist.barrier()
        e_ms = (ev0.elapsed_time(ev1) if use_cuda else e_wall * 1e3) / args.steps
        # the host must be able to keep up too: take the slower of device and wall clock
        e_ms = max(e_ms, e_wall * 1e3 / args.steps)
        t_e = torch.tensor([e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t_e, op=dist.ReduceOp.MAX)
        e_ms = float(t_e.item())
        assert bool(torch.isfinite(loss_host).all()), "non-finite loss in the end-to-end arm"
        e2e = {"value": per_gpu * world / (e_ms / 1e3), "unit": desc["unit"], "ms_per_step": e_ms,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4, "last_loss": float(loss_host[-1])}
        trainer.check()

    clocks = sampler.stop() if sampler else None

    # ---- what ran, and what it left exposed (untimed extras, after the measured regions) ----
    state = trainer.state
    engines = list(getattr(state, "_engines", {}).values()) if state is not None else []
    backends = sorted({(e.symm.backend if e.symm is not None else ("nccl" if e.world > 1 else "local"))
                       for e in engines}) or (["library all-reduce (no native engine ran)"] if world > 1 else ["none"])
    graph_replays = sum(int(getattr(e.exec_plan, "graph_replays", 0) or 0) for e in engines
                        if getattr(e, "exec_plan", None) is not None)
    fused = [bool(getattr(e, "fused", False)) for e in engines]
    phase_ms = exposed_ms = bypass_ms = None
    if state is not None and use_cuda and args.impl == "ours":
        state.enable_phase_timing()
        for i in range(3):
            trainer.step(*dev_batches[i % nbuf])
        summary = state.phase_summary()
        state.enable_phase_timing(False)
        phase_ms = {k: round(v["ms"] / 3, 4) for k, v in summary.items()}     # per step, all buckets
    if state is not None and args.impl in ("ours", "restated"):
        from conef_b200.parallel import hooks as _hooks
        _hooks.BYPASS = True            # hooks return their bucket untouched: a step without compression or comm
        for i in range(2):
            trainer.step(*dev_batches[i % nbuf])
        bypass_ms, _ = timed_steps(args.steps)
        _hooks.BYPASS = False
        exposed_ms = ms - bypass_ms

    if rank == 0:
        out = {
            "metric": f"{desc['unit']} training throughput, {desc['model']}, {desc['reducer']}",
            "value": value, "unit": desc["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": desc["dtype"], "data": "synthetic (random-init weights, N(0,1) / uniform-id inputs)",
            "impl": args.impl,
            "config": {"model": desc["model"], "global_batch": per_gpu * world, "per_gpu_batch": per_gpu,
                       "seq_len": desc.get("seq_len"), "parallelism": f"dp{world}", "reducer": ns.grad_reducer,
                       "rank": ns.matrix_approximation_rank, "sketch_size": ns.sketch_size, "beta": ns.beta,
                       "l2": "256 MB buffer written between timed steps (outside the per-step event pair)",
                       "timing": "CUDA events per step on the launching stream, mean over steps, max over ranks",
                       "comm": os.environ.get("CONEF_COMM", "auto"), "bucket_cap_mb": tkw.get("bucket_cap_mb", 25.0), "tc": os.environ.get("CONEF_TC", "1"),
                       "cuda_graph_blocks": int(getattr(trainer, "graphed_modules", 0)),
                       "cudnn_autotune": bool(tkw.get("cudnn_autotune", False))},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
            "wall_s_timed_region": wall,
            "ef_buffer_mb": (state.ef_buffer_bytes() / 1e6) if state is not None else 0.0,
            # the data plane that actually ran (not the request): symm / ipc = own kernels over peer
            # memory, local = one rank, nccl = library all-reduce
            "comm_backend_used": backends, "graph_replays": graph_replays,
            "buckets": len(engines), "buckets_on_fused_pipeline": sum(fused),
            # step time minus the time of the same step with the hooks returning at once (same process)
            "exposed_comm_ms": exposed_ms, "ms_per_step_hooks_bypassed": bypass_ms,
            "phase_ms": phase_ms,
        }
        if state is not None and hasattr(state, "compression_stats"):
            out["compression_rate"] = state.compression_stats()[0]
        if state is not None:
            out["wire_mb_per_step_per_rank"] = state.wire_bytes_per_step() / 1e6
        os.write(real_stdout, (json.dumps(out) + "\n").encode())
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
