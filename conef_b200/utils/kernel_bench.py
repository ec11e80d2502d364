"""Micro-benchmark of the compression kernels in isolation, with roofline fractions.

    python -m conef_b200.utils.kernel_bench --case wrn --iters 20
    python -m conef_b200.utils.kernel_bench --case bert --only decompress --iters 3     # small, for ncu

Builds one synthetic gradient "bucket" larger than the 126 MB L2 (so that DRAM figures
mean something), runs every kernel of the PowerSGD + ConEF pipeline and of the
random-block pipeline on it, times each with CUDA events on the launching stream (warm-up,
synchronise on both sides) and reports achieved bytes/s against the measured HBM copy
bandwidth (``MEASURED_PEAKS.json`` next to the repository root when present, else the
6.65 TB/s fallback).  Algorithmic bytes are the minimum traffic of each kernel: every
matrix element read (and written, where the kernel rewrites it) once.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import numpy as np
import torch

import conef_b200 as cb
from conef_b200.ops import native
from conef_b200.parallel.engine import PowerSGDEngine, RandBlockEngine

CASES = {
    # (shapes, rank): matrices as in the named model, repeated until the bucket exceeds L2
    "wrn": ([(640, 640, 3, 3)] * 10 + [(640,)] * 10 + [(320, 320, 3, 3)] * 6 + [(100, 640), (100,)], 4),
    "bert": ([(1024, 1024)] * 24 + [(4096, 1024)] * 8 + [(1024, 4096)] * 8 + [(1024,)] * 16 + [(4096,)] * 8, 8),
    # the LSTM language model: row pitch 650 * 4 bytes, which only the folded view can give to TMA
    "lstm": ([(33278, 650)] + [(2600, 650)] * 24 + [(2600,)] * 12, 4),
    # Transformer-base: attention / feed-forward matrices and one embedding; `--only phase` runs it with
    # the hPowerSGD hook and the low-rank error store of that benchmark configuration
    "transformer": ([(512, 512)] * 48 + [(2048, 512)] * 12 + [(512, 2048)] * 12 + [(32000, 512)] + [(512,)] * 60, 8),
    "small": ([(256, 1024), (64,), (640, 360)], 4),
}


class _Bucket:
    def __init__(self, shapes, device):
        total = sum(int(np.prod(s)) for s in shapes)
        self.buf = torch.randn(total, device=device)
        self.shapes = shapes

    def buffer(self):
        return self.buf

    def index(self):
        return 0

    def is_last(self):
        return True

    def gradients(self):
        out, off = [], 0
        for s in self.shapes:
            n = int(np.prod(s))
            out.append(self.buf[off : off + n].view(s))
            off += n
        return out


def _peak_gbs() -> tuple:
    for cand in (Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json",):
        if cand.exists():
            return float(json.loads(cand.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _time(fn, iters, warmup=3, prep=None):
    """Median device time of ``fn``; ``prep`` (untimed) restores the inputs before every call."""
    for _ in range(warmup):
        if prep is not None:
            prep()
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for s, e in ev:
        if prep is not None:
            prep()
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    ts = sorted(s.elapsed_time(e) for s, e in ev)
    return ts[len(ts) // 2] * 1e-3          # median, seconds


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="wrn", choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default=None, help="run only kernels whose name contains this")
    ap.add_argument("--sketch-size", type=float, default=0.1)
    args = ap.parse_args()

    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29655")
    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    shapes, rank = CASES[args.case]
    bucket = _Bucket(shapes, dev)
    buf = bucket.buffer()
    peak, peak_kind = _peak_gbs()
    group = dist.group.WORLD
    st = native.stream_ptr(dev)
    lib = native.lib()
    rows = []

    def record(name, seconds, nbytes, note=""):
        gbs = nbytes / seconds / 1e9
        rows.append((name, seconds * 1e6, nbytes / 1e6, gbs, gbs / peak, note))

    def want(name):
        return args.only is None or args.only in name

    # ---------------- PowerSGD + ConEF sketch pipeline ----------------
    for tc in ("1", "0"):
        os.environ["CONEF_TC"] = tc
        state = cb.PowerSGDState(None, matrix_approximation_rank=rank, start_powerSGD_iter=2,
                                 use_error_compression=True, sketch_size=args.sketch_size)
        eng = PowerSGDEngine(state, buf, bucket.gradients(), group, "powersgd")
        plan = eng.plan
        mat_bytes = 4 * sum(e.numel for e in plan.mats)
        sk_bytes = 4 * eng.sketch_arena.numel()
        pmem = torch.randn(plan.total_p, device=dev)
        qz = eng.qz
        qz.normal_()
        qmem = qz[: plan.total_q]
        eng.sketch_arena.normal_()
        tag = "tc" if eng.use_tc else "simt"
        if tc == "1" and not eng.use_tc:
            continue
        if want(f"p_{tag}"):
            def run_p():
                qz[plan.total_q :].zero_()
                native.check(lib.conef_sketch_project(eng.mats_dev.data_ptr(), eng.nm, eng.max_cols,
                                                      eng.tables.data_ptr(), qz.data_ptr(), 0.1, 0, st))
                pmem.zero_()
                eng._launch_p(buf.data_ptr(), eng.aux_ptr, qz, pmem, st)
            t = _time(run_p, args.iters)
            record(f"p_{tag}: P=GQ+S(aH^TQ)", t, mat_bytes + sk_bytes, "read G and the sketch once, nothing written back")
        if want(f"q_{tag}"):
            def run_q():
                qz.zero_()
                eng._launch_q(buf.data_ptr(), eng.aux_ptr, pmem, qz, st)
                native.check(lib.conef_sketch_project(eng.mats_dev.data_ptr(), eng.nm, eng.max_cols,
                                                      eng.tables.data_ptr(), qz.data_ptr(), 0.1, 1, st))
            t = _time(run_q, args.iters)
            record(f"q_{tag}: Q=G^TP+aH(S^TP)", t, mat_bytes + sk_bytes, "read G and the sketch once")
        if tc == "1" and want("phase"):
            # the three phases of a whole hook call, every launch they need included (executor, direct
            # launches; CUDA events around each phase on the hook's stream)
            for fused in ("1", "0"):
                os.environ["CONEF_FUSED"] = fused
                if args.case == "transformer":
                    st2 = cb.hPowerSGDState(None, matrix_approximation_rank=rank, start_powerSGD_iter=2,
                                            use_error_compression=True, error_compressor="lowrank", error_rank=rank)
                else:
                    st2 = cb.PowerSGDState(None, matrix_approximation_rank=rank, start_powerSGD_iter=2,
                                           use_error_compression=True, sketch_size=args.sketch_size)
                st2.iter = 2
                for _ in range(3):
                    cb.powerSGD_hook(st2, bucket).wait()
                torch.cuda.synchronize()
                st2.enable_phase_timing()
                for _ in range(args.iters):
                    cb.powerSGD_hook(st2, bucket).wait()
                torch.cuda.synchronize()
                e2 = st2._engines[0]
                label = f"fused, {e2.exec_plan.launched} launches in D" if e2.fused else "long form"
                algo = {"psgd/P=GQ": mat_bytes + sk_bytes, "psgd/reduce+orth+Q=GtP": mat_bytes + sk_bytes,
                        "psgd/reduce+decompress": 2 * mat_bytes + 2 * sk_bytes}
                for name, rec in st2.phase_summary().items():
                    record(f"phase {name} [{'fused' if e2.fused else 'long'}]", rec["ms_per_call"] * 1e-3,
                           algo.get(name, mat_bytes), label)
            os.environ.pop("CONEF_FUSED", None)
        if tc == "1":
            continue
        if want("orth"):
            def run_orth():
                eng.pu.normal_()
                eng._orth(0, "grad", eng.pu, 0.0, st)
            t = _time(run_orth, args.iters)
            record("orthogonalize(P)", t, 24 * plan.total_p, "3 row-parallel passes over P (read + write)")
        if want("decompress"):
            t = _time(lambda: native.check(lib.conef_psgd_decompress(
                eng.mats_dev.data_ptr(), eng.d_tiles.data_ptr(), eng.n_d_tiles, eng.d_nblk, eng.d_rbu, eng.d_rows, buf.data_ptr(),
                pmem.data_ptr(), qmem.data_ptr(), 1.0, eng.sketch_arena.data_ptr(), eng.tables.data_ptr(),
                eng.counts.data_ptr(), 0, 0.1, 0.9, native.EF_SKETCH, eng.max_rank, eng.d_smem,
                eng.status.data_ptr(), st)), args.iters)
            record("decompress+sketch update", t, 2 * mat_bytes + 2 * sk_bytes,
                   "read M, write M_hat, r/w sketch")
        if want("decompress"):      # (this part of the loop runs once, in the second iteration)
            # dense error feedback and no error feedback: the column-order kernel (no sketch, no atomics)
            state_d = cb.PowerSGDState(None, matrix_approximation_rank=rank, start_powerSGD_iter=2, use_error_feedback=True)
            eng_d = PowerSGDEngine(state_d, buf, bucket.gradients(), group, "powersgd")
            err = torch.zeros_like(buf)
            for mode, nb, what in ((native.EF_DENSE, 4 * mat_bytes, "read M and the error, write M_hat and the error"),
                                   (native.EF_NONE, mat_bytes, "write M_hat")):
                t = _time(lambda: native.check(lib.conef_psgd_decompress(
                    eng_d.mats_dev.data_ptr(), eng_d.d_tiles.data_ptr(), eng_d.n_d_tiles, 0, 1, eng_d.d_rows,
                    buf.data_ptr(), pmem.data_ptr(), qmem.data_ptr(), 1.0, 0, 0, 0, err.data_ptr(), 1.0, 1.0, mode,
                    eng_d.max_rank, 0, eng_d.status.data_ptr(), st)), args.iters)
                record("decompress, dense error feedback" if mode == native.EF_DENSE else "decompress, no error feedback",
                       t, nb, what)
            del err, eng_d, state_d
        if want("segments"):
            t = _time(lambda: native.check(lib.conef_gather_segments(
                eng.segs_dev.data_ptr(), len(plan.segs), buf.data_ptr(), 0, eng.staging.data_ptr(), plan.total_unc,
                st)), args.iters)
            record("gather_segments", t, 8 * plan.total_unc, "latency bound (small)")
        # whole hook, one bucket
        if want("hook"):
            state.iter = 2
            t = _time(lambda: cb.powerSGD_hook(state, bucket).wait(), args.iters)
            record("powerSGD_hook (whole bucket, ws=1)", t, 4 * mat_bytes + 4 * sk_bytes,
                   "ideal: G read by P, Q and decompress, written once; sketch read 3x, written once")

    os.environ["CONEF_TC"] = "1"

    # ---------------- random block pipeline ----------------
    for kind, kw in (("ef", dict()), ("sketch", dict(use_error_compression=True, sketch_size=args.sketch_size)),
                     ("quant8", dict(use_error_compression=True, error_compressor="quant8", beta=0.0))):
        if not want(f"randblock_{kind}"):
            continue
        state = cb.RandomBlockState(None, start_compression_iter=2, compression_ratio=0.1, **kw)
        state.iter = 2
        nbytes = 4 * sum(int(np.prod(s)) for s in shapes if len(s) > 1)
        fresh = buf.clone()
        refill = lambda: buf.copy_(fresh)       # the hook zeroes what it does not send
        t = _time(lambda: cb.RandomBlock_hook(state, bucket).wait(), args.iters, prep=refill)
        per = {"ef": 4.0, "sketch": 2.2, "quant8": 2.5}[kind]      # passes over the tensors (r/w gradient + error store)
        record(f"RandomBlock_hook {kind} (whole bucket, ws=1)", t, per * nbytes, "gather+error update, scatter")
        # the two kernels alone (the hook also draws the block offsets on the host and uploads them)
        eng = state._engines[0]
        beta = getattr(state, "beta", 0.0)
        sk = native.ptr(eng.err_arena) if eng.ef_mode == native.EF_SKETCH else 0
        de = native.ptr(eng.err_arena) if eng.ef_mode == native.EF_DENSE else 0
        t = _time(lambda: native.check(lib.conef_randblock_gather(
            eng.blks_dev.data_ptr(), eng.tiles.data_ptr(), eng.n_tiles, eng.nblk_tiles, eng.rows, buf.data_ptr(),
            eng.staging_blk.data_ptr(), 1.0, sk, native.ptr(eng.tables), native.ptr(eng.counts), de,
            native.ptr(eng.codes), native.ptr(eng.scales), 1.0 - beta, beta, eng.ef_mode, eng.smem, st)), args.iters,
            prep=refill)
        record(f"  randblock_gather kernel {kind}", t, (per - 0.2) * nbytes, "read G (+ error), write G / block, update error")
        t = _time(lambda: native.check(lib.conef_randblock_scatter(
            eng.blks_dev.data_ptr(), len(eng.plan.blocks), buf.data_ptr(), 0, 1, eng.staging_blk.data_ptr(), 1.0,
            eng.plan.total_block, st)), args.iters)
        record(f"  randblock_scatter kernel {kind}", t, 0.2 * nbytes, "read block, write block")

    # ---------------- hPowerSGD top-k error store ----------------
    if want("topk"):
        state = cb.hPowerSGDState(None, matrix_approximation_rank=rank, start_powerSGD_iter=2,
                                  use_error_compression=True, topk_ratio=0.4)
        eng = PowerSGDEngine(state, buf, bucket.gradients(), group, "powersgd")
        eng.topk_arena.normal_()
        mat_bytes = 4 * sum(e.numel for e in eng.plan.mats)
        t = _time(lambda: native.check(lib.conef_topk_keep(
            eng.mats_dev.data_ptr(), eng.nm, eng.topk_tiles.data_ptr(), eng.n_topk_tiles, eng.topk_arena.data_ptr(),
            0.4, eng.topk_scratch.data_ptr(), st)), args.iters)
        record("topk_keep (radix select, all matrices)", t, 4.8 * mat_bytes,
               "3 histogram reads + prune (read, ~80 % written back)")
        state.iter = 2
        t = _time(lambda: cb.hpowerSGD_hook(state, bucket).wait(), args.iters)
        record("hpowerSGD_hook top-k (whole bucket, ws=1)", t, (3 * 2 + 2 + 4.8) * mat_bytes,
               "G and E read by P, Q, decompress; M_hat and E written; top-k")

    # ---------------- model-side column kernels (bias gradient, batch norm) ----------------
    if want("colsum"):
        from conef_b200.ops import colsum
        # a channels-last bf16 activation larger than L2: WRN-28-10's first stage at four times its batch
        x = torch.randn(512, 160, 32, 32, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        dy = torch.randn_like(x)
        nb = x.numel() * 2
        w = torch.rand(160, device=dev) + 0.5
        b = torch.randn(160, device=dev)
        mean, invstd = colsum.channel_stats(x, 1e-5)
        sums = colsum.channel_dot_relu(dy, x, mean, invstd, w, b)
        cnt = torch.full((1,), x.numel() // 160, dtype=torch.int32, device=dev)
        record("channel_sum (bias gradient)", _time(lambda: colsum.channel_sum(dy), args.iters), nb, "read dy")
        record("  torch: dy.sum((0, 2, 3))", _time(lambda: dy.sum(dim=(0, 2, 3)), args.iters), nb, "library")
        record("channel_stats (batch-norm statistics)", _time(lambda: colsum.channel_stats(x, 1e-5), args.iters), nb, "read x")
        record("  torch: batch_norm_stats", _time(lambda: torch.batch_norm_stats(x, 1e-5), args.iters), nb, "library")
        record("bn_apply + ReLU", _time(lambda: colsum.bn_apply(x, mean, invstd, w, b, True), args.iters), 2 * nb,
               "read x, write y")
        record("  torch: batch_norm_elemt, relu", _time(lambda: torch.relu(torch.batch_norm_elemt(x, w, b, mean, invstd, 1e-5)),
                                                       args.iters), 4 * nb, "library: two passes")
        record("channel_dot_relu (backward sums)", _time(lambda: colsum.channel_dot_relu(dy, x, mean, invstd, w, b), args.iters),
               2 * nb, "read dy and x")
        record("  torch: batch_norm_backward_reduce", _time(lambda: torch.batch_norm_backward_reduce(dy, x, mean, invstd, w, True, True, True),
                                                           args.iters), 2 * nb, "library (no ReLU mask)")
        record("bn_backward_apply + ReLU", _time(lambda: colsum.bn_backward_apply(dy, x, mean, invstd, w, b, sums[0], sums[1], True),
                                                 args.iters), 3 * nb, "read dy and x, write dx")
        record("  torch: batch_norm_backward_elemt", _time(lambda: torch.batch_norm_backward_elemt(dy, x, mean, invstd, w, sums[0], sums[1], cnt),
                                                          args.iters), 3 * nb, "library (no ReLU mask)")
        y = x.clone()
        record("bias_add_", _time(lambda: colsum.bias_add_(y, b), args.iters), 2 * nb, "read and write y")
        record("  torch: y += bias", _time(lambda: y.add_(b.to(y.dtype).view(1, -1, 1, 1)), args.iters), 2 * nb, "library")
        del x, dy, y

    # ---------------- LAMB ----------------
    if want("lamb"):
        from conef_b200.optim import FusedLAMB
        ps = [torch.nn.Parameter(torch.randn(s, device=dev)) for s in shapes]
        for p in ps:
            p.grad = torch.randn_like(p)
        opt = FusedLAMB(ps, lr=1e-3)
        n = sum(p.numel() for p in ps)
        t = _time(opt.step, args.iters)
        record("FusedLAMB.step", t, 4 * n * (1 + 7 + 3), "gnorm r, stage1 r4 w3, stage2 r2 w1")

    print(f"case={args.case} bucket={buf.numel() * 4 / 1e6:.1f} MB rank={rank} peak={peak:.0f} GB/s ({peak_kind})")
    print(f"{'kernel':44s} {'us':>9s} {'MB':>9s} {'GB/s':>8s} {'of ' + peak_kind:>12s}  note")
    for name, us, mb, gbs, frac, note in rows:
        print(f"{name:44s} {us:9.1f} {mb:9.1f} {gbs:8.0f} {frac:12.2f}  {note}")


if __name__ == "__main__":
    main()
