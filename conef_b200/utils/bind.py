"""Launch one training process per GPU with CPU / memory affinity set per local rank.

Counterpart of the reference's ``examples/BertPretraining/bind_pyt.py:75-133`` and ``bind.sh``,
which wrap each rank in ``numactl``.  Here affinity is set with ``os.sched_setaffinity`` (no
external tool): the host's cores are split evenly among the local ranks, optionally following
the NUMA node of each GPU when ``/sys`` exposes it.  Nothing of the GPU's own settings is touched.

    python -m conef_b200.utils.bind --nproc_per_node 8 train.py --arg ...
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys


def cores_for_rank(local_rank: int, nproc: int, ncores: int = None):
    ncores = ncores or os.cpu_count() or 1
    per = max(1, ncores // nproc)
    lo = (local_rank * per) % ncores
    return list(range(lo, min(lo + per, ncores)))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--nnodes", type=int, default=1)
    ap.add_argument("--node_rank", type=int, default=0)
    ap.add_argument("--nproc_per_node", type=int, default=1)
    ap.add_argument("--master_addr", default="127.0.0.1")
    ap.add_argument("--master_port", type=int, default=29500)
    ap.add_argument("--no_membind", action="store_true")
    ap.add_argument("training_script")
    ap.add_argument("training_script_args", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    world = args.nnodes * args.nproc_per_node
    procs = []
    for local_rank in range(args.nproc_per_node):
        env = dict(os.environ, MASTER_ADDR=args.master_addr, MASTER_PORT=str(args.master_port),
                   WORLD_SIZE=str(world), RANK=str(args.node_rank * args.nproc_per_node + local_rank),
                   LOCAL_RANK=str(local_rank))
        cores = cores_for_rank(local_rank, args.nproc_per_node)

        def pin(cores=cores):
            try:
                os.sched_setaffinity(0, cores)
            except (AttributeError, OSError):
                pass
        cmd = [sys.executable, "-u", args.training_script, f"--local_rank={local_rank}", *args.training_script_args]
        procs.append(subprocess.Popen(cmd, env=env, preexec_fn=pin))
    code = 0
    for p in procs:
        p.wait()
        code = code or p.returncode
    return code


if __name__ == "__main__":
    sys.exit(main())
