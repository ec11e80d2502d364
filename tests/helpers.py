"""Test helpers: fake DDP buckets and a gloo process launcher."""
import os
import socket
import traceback

import torch
import torch.multiprocessing as mp


class FakeBucket:
    """Duck-typed stand-in for ``dist.GradBucket``: a flat buffer plus views."""

    def __init__(self, shapes, index=0, last=True, device="cpu", seed=0, dtype=torch.float32):
        g = torch.Generator().manual_seed(seed)
        total = sum(int(torch.Size(s).numel()) for s in shapes)
        self._buf = torch.randn(total, generator=g, dtype=dtype).to(device)
        self._shapes = [tuple(s) for s in shapes]
        self._index, self._last = index, last

    def buffer(self):
        return self._buf

    def index(self):
        return self._index

    def is_last(self):
        return self._last

    def gradients(self):
        out, off = [], 0
        for s in self._shapes:
            n = int(torch.Size(s).numel())
            out.append(self._buf[off : off + n].view(s))
            off += n
        return out

    def clone(self, device=None):
        other = FakeBucket.__new__(FakeBucket)
        other._buf = self._buf.clone() if device is None else self._buf.to(device).clone()
        other._shapes, other._index, other._last = self._shapes, self._index, self._last
        return other

    def refill(self, seed):
        g = torch.Generator().manual_seed(seed)
        self._buf.copy_(torch.randn(self._buf.numel(), generator=g))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, backend, fn, args, errq):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world=2, args=(), backend="gloo", timeout=240):
    """Run ``fn(rank, world, *args)`` in ``world`` spawned processes; raises on any failure."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, backend, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    if alive or msgs or any(p.exitcode != 0 for p in procs):
        raise AssertionError(f"ranks failed (alive={len(alive)}, exit={[p.exitcode for p in procs]}):\n" +
                             "\n".join(f"[rank {r}] {m}" for r, m in msgs))
