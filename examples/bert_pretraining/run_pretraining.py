#!/usr/bin/env python
"""BERT pre-training (masked LM + next-sentence prediction) with compressed gradients.

Counterpart of the reference's ``examples/BertPretraining/run_pretraining_conef.py``:
``--grad_reducer / --start_compression_percentage / --compression_ratio / --sketch_size / --beta``,
LAMB with linear warm-up, gradient accumulation, optional activation checkpointing, periodic
checkpoints that keep the three most recent files, resume from the newest checkpoint, SIGTERM
turned into "checkpoint and exit", throughput summary in sequences per second.

Execution modes, as in the reference (``run_pretraining_conef.py:356-404,492-499``):
* one process per GPU under ``torchrun`` / ``torch.distributed.run``: DistributedDataParallel with
  the compression hook of ``--grad_reducer`` (default);
* ``--allreduce_post_accumulation`` (optionally ``--allreduce_post_accumulation_fp16``): no DDP and
  no hook; gradients accumulate locally and are all-reduced once per optimizer step as one flat
  buffer (forced off when ``--gradient_accumulation_steps 1``);
* ``--local_rank -1``: a single process without a process group, ``torch.nn.DataParallel`` over
  all visible GPUs when there are several.

Differences: bf16 autocast instead of apex amp, the in-tree multi-tensor LAMB instead of apex
FusedLAMB, synthetic shards instead of HDF5 files (no h5py / corpus on the box), and the reducer's
state (error buffers, sketches, P/Q memory, RNG) is part of every checkpoint, which the reference omits.
"""
import argparse
import contextlib
import os
import sys
import time

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP
from torch.utils.data import DataLoader

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import conef_b200 as cb  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.data import ShardPrefetcher, SyntheticBertShard, shard_files  # noqa: E402
from conef_b200.optim import FusedLAMB, LinearWarmUpScheduler  # noqa: E402
from conef_b200.parallel.accumulate import PostAccumulationAllReduce, broadcast_parameters  # noqa: E402
from conef_b200.utils import (GracefulStop, JsonLogger, latest_checkpoint, load_checkpoint,  # noqa: E402
                              save_checkpoint)


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--config_file", default=None, help="BertConfig JSON; BERT-large when omitted")
    p.add_argument("--bert_model", default="large", choices=["large", "base", "tiny"])
    p.add_argument("--output_dir", default="results/bert")
    p.add_argument("--max_seq_length", type=int, default=128)
    p.add_argument("--max_predictions_per_seq", type=int, default=20)
    p.add_argument("--train_batch_size", type=int, default=64, help="per process, per optimizer step")
    p.add_argument("--gradient_accumulation_steps", type=int, default=1)
    p.add_argument("--learning_rate", type=float, default=1.25e-3)
    p.add_argument("--warmup_proportion", type=float, default=0.01)
    p.add_argument("--max_steps", type=int, default=20)
    p.add_argument("--steps_this_run", type=int, default=-1)
    p.add_argument("--num_steps_per_checkpoint", type=int, default=100)
    p.add_argument("--resume_from_checkpoint", action="store_true")
    p.add_argument("--init_checkpoint", default=None,
                   help="checkpoint file or directory (its latest checkpoint) whose model weights start a new run, "
                        "e.g. phase 2 from the end of phase 1; optimizer, schedule and reducer state start fresh")
    p.add_argument("--checkpoint_activations", action="store_true")
    p.add_argument("--bf16", action="store_true", default=True)
    p.add_argument("--input_dir", default=None,
                   help="directory of .npz shards written by create_pretraining_data.py; synthetic shards when omitted")
    p.add_argument("--shard_size", type=int, default=2048, help="synthetic instances per shard")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--grad_reducer", default="conef_powersgd", choices=cb.REDUCERS)
    p.add_argument("--start_compression_percentage", type=float, default=0.1)
    p.add_argument("--compression_ratio", type=float, default=0.1)
    p.add_argument("--sketch_size", type=float, default=0.1)
    p.add_argument("--beta", type=float, default=0.9)
    p.add_argument("--matrix_approximation_rank", type=int, default=8)
    p.add_argument("--min_compression_rate", type=float, default=2)
    p.add_argument("--orthogonalization_epsilon", type=float, default=0)
    p.add_argument("--error_compressor", default=None)
    p.add_argument("--allreduce_post_accumulation", action="store_true",
                   help="accumulate locally, all-reduce all gradients once per optimizer step (no DDP, no hook)")
    p.add_argument("--allreduce_post_accumulation_fp16", action="store_true",
                   help="do that all-reduce in fp16")
    p.add_argument("--local_rank", type=int, default=int(os.environ.get("LOCAL_RANK", 0)),
                   help="-1: single process, torch.nn.DataParallel over the visible GPUs")
    args = p.parse_args()
    args.start_compression_iter = max(2, int(args.max_steps * args.start_compression_percentage))
    if args.local_rank == -1 or args.gradient_accumulation_steps == 1:
        args.allreduce_post_accumulation = args.allreduce_post_accumulation_fp16 = False
    if args.gradient_accumulation_steps < 1 or args.train_batch_size % args.gradient_accumulation_steps:
        raise ValueError("--train_batch_size must be a positive multiple of --gradient_accumulation_steps")
    return args


def build_model(args):
    if args.config_file:
        cfg = models.BertConfig.from_json_file(args.config_file)
    elif args.bert_model == "large":
        cfg = models.BertConfig.large()
    elif args.bert_model == "base":
        cfg = models.BertConfig.base()
    else:
        cfg = models.BertConfig(30528, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512)
    if cfg.vocab_size % 8 != 0:                 # pad the vocabulary to a multiple of 8, as the reference does
        cfg.vocab_size += 8 - cfg.vocab_size % 8
    net = models.BertForPreTraining(cfg)
    net.bert._checkpoint_activations = args.checkpoint_activations
    return net, cfg


def main():
    args = parse()
    distributed = args.local_rank != -1
    rank, world = (int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))) if distributed else (0, 1)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29504")
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", max(args.local_rank, 0)) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    if distributed:
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    torch.manual_seed(args.seed + rank)
    net, cfg = build_model(args)
    net = net.to(device)
    decay = [p for n, p in net.named_parameters() if p.dim() > 1]
    no_decay = [p for n, p in net.named_parameters() if p.dim() <= 1]
    opt = FusedLAMB([{"params": decay, "weight_decay": 0.01}, {"params": no_decay, "weight_decay": 0.0}],
                    lr=args.learning_rate)
    sched = LinearWarmUpScheduler(opt, warmup=args.warmup_proportion, total_steps=args.max_steps)
    state, post = None, None
    if distributed and not args.allreduce_post_accumulation:
        ddp = DDP(net, device_ids=[args.local_rank] if cuda else None, gradient_as_bucket_view=True)
        state = cb.get_comm_hooks(args, ddp, args.local_rank)
    elif distributed:
        # no DDP: same start on every rank, one flat all-reduce per optimizer step
        broadcast_parameters(net)
        post = PostAccumulationAllReduce(
            net.parameters(), wire_dtype=torch.float16 if args.allreduce_post_accumulation_fp16 else torch.float32)
        ddp = net
    else:
        ddp = torch.nn.DataParallel(net) if cuda and torch.cuda.device_count() > 1 else net
    no_sync = ddp.no_sync if isinstance(ddp, DDP) else contextlib.nullcontext
    crit = models.BertPretrainingCriterion(cfg.vocab_size)
    global_step, epoch = 0, 0
    resumed = False
    if args.resume_from_checkpoint:
        ck = latest_checkpoint(args.output_dir)
        if ck:
            info = load_checkpoint(ck, model=ddp, optimizer=opt, reducer_state=state, device=device, rank=rank)
            global_step, epoch = info["step"], info["extra"].get("epoch", 0)
            resumed = True
    if args.init_checkpoint and not resumed:
        ck = latest_checkpoint(args.init_checkpoint) if os.path.isdir(args.init_checkpoint) else args.init_checkpoint
        if not ck or not os.path.exists(ck):
            raise FileNotFoundError(f"--init_checkpoint {args.init_checkpoint}: no checkpoint found")
        load_checkpoint(ck, model=ddp, device=device, rank=rank)          # weights only
    if rank == 0:
        os.makedirs(args.output_dir, exist_ok=True)
    stop, log = GracefulStop(), JsonLogger(os.path.join(args.output_dir, "log.jsonl") if rank == 0 else None)
    micro = args.train_batch_size // args.gradient_accumulation_steps
    steps_this_run = args.steps_this_run if args.steps_this_run > 0 else args.max_steps
    done, t_start, seqs, skipped_steps = 0, time.time(), 0, 0
    amp = torch.autocast("cuda", dtype=torch.bfloat16) if (cuda and args.bf16) else torch.autocast("cpu", enabled=False)
    ddp.train()
    def epoch_shards(epoch):
        """This rank's shards of an epoch; files are read one shard ahead in the background."""
        if args.input_dir:
            pre = ShardPrefetcher(shard_files(args.input_dir, rank, world, epoch, args.seed),
                                  args.max_predictions_per_seq)
            yield from pre
            pre.close()
        else:
            yield SyntheticBertShard(args.shard_size, args.max_seq_length, 30522, args.max_predictions_per_seq,
                                     seed=args.seed + 1000 * epoch + rank)

    def batches(epoch):
        for shard in epoch_shards(epoch):
            yield from DataLoader(shard, micro, shuffle=True, num_workers=0 if args.input_dir else 2,
                                  pin_memory=cuda, drop_last=len(shard) >= micro)

    while done < steps_this_run and global_step < args.max_steps and not stop.requested:
        for it, batch in enumerate(batches(epoch)):
            ids, seg, mask, labels, nsp = (t.to(device, non_blocking=True) for t in batch)
            sync = (it + 1) % args.gradient_accumulation_steps == 0
            with (no_sync() if not sync else contextlib.nullcontext()), amp:
                loss = crit(ddp(ids, seg, mask), (labels, nsp)) / args.gradient_accumulation_steps
            with (no_sync() if not sync else contextlib.nullcontext()):
                loss.backward()
            seqs += ids.size(0)
            if not sync:
                continue
            sched.step()
            if post is not None and not post.allreduce():
                skipped_steps += 1                # a non-finite value came out of the fp16 all-reduce
                opt.zero_grad(set_to_none=False)
                continue
            opt.step()
            opt.zero_grad(set_to_none=False)
            global_step += 1
            done += 1
            if global_step % 10 == 0 or done == steps_this_run:
                log.log(global_step, loss=float(loss) * args.gradient_accumulation_steps, lr=opt.param_groups[0]["lr"])
            if global_step % args.num_steps_per_checkpoint == 0 or stop.requested:
                save_checkpoint(args.output_dir, global_step, model=ddp, optimizer=opt, reducer_state=state,
                                extra={"epoch": epoch, "per_rank": True}, rank=rank)
            if done >= steps_this_run or global_step >= args.max_steps or stop.requested:
                break
        epoch += 1
    if cuda:
        torch.cuda.synchronize()
    if state is not None:
        state.check_status()
    dt = time.time() - t_start
    save_checkpoint(args.output_dir, global_step, model=ddp, optimizer=opt, reducer_state=state,
                    extra={"epoch": epoch, "per_rank": True}, rank=rank)
    final = torch.tensor([float(loss) * args.gradient_accumulation_steps], device=device)
    if distributed:
        dist.all_reduce(final)
    mode = "ddp+hook" if isinstance(ddp, DDP) else "post-accumulation all-reduce" if post is not None else \
        "data-parallel (one process)" if isinstance(ddp, torch.nn.DataParallel) else "single device"
    log.log("summary", training_sequences_per_second=seqs * world / dt, final_loss=float(final) / world,
            ef_buffer_mb=(state.ef_buffer_bytes() / 1e6) if state else 0.0, mode=mode, skipped_steps=skipped_steps,
            allreduce_mb_per_step=(post.bytes_on_wire / 1e6) if post is not None else None)
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
