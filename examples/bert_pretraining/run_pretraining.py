#!/usr/bin/env python
"""BERT pre-training (masked LM + next-sentence prediction) with compressed gradients.

Counterpart of the reference's ``examples/BertPretraining/run_pretraining_conef.py``:
``--grad_reducer / --start_compression_percentage / --compression_ratio / --sketch_size / --beta``,
LAMB with linear warm-up, gradient accumulation, optional activation checkpointing, periodic
checkpoints that keep the three most recent files, resume from the newest checkpoint, SIGTERM
turned into "checkpoint and exit", throughput summary in sequences per second.

Differences: bf16 autocast instead of apex amp, the in-tree multi-tensor LAMB instead of apex
FusedLAMB, synthetic shards instead of HDF5 files (no h5py / corpus on the box), and the reducer's
state (error buffers, sketches, P/Q memory, RNG) is part of every checkpoint, which the reference omits.
"""
import argparse
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
    p.add_argument("--local_rank", type=int, default=int(os.environ.get("LOCAL_RANK", 0)))
    args = p.parse_args()
    args.start_compression_iter = max(2, int(args.max_steps * args.start_compression_percentage))
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
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29504")
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", args.local_rank) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    torch.manual_seed(args.seed + rank)
    net, cfg = build_model(args)
    net = net.to(device)
    decay = [p for n, p in net.named_parameters() if p.dim() > 1]
    no_decay = [p for n, p in net.named_parameters() if p.dim() <= 1]
    opt = FusedLAMB([{"params": decay, "weight_decay": 0.01}, {"params": no_decay, "weight_decay": 0.0}],
                    lr=args.learning_rate)
    sched = LinearWarmUpScheduler(opt, warmup=args.warmup_proportion, total_steps=args.max_steps)
    ddp = DDP(net, device_ids=[args.local_rank] if cuda else None, gradient_as_bucket_view=True)
    state = cb.get_comm_hooks(args, ddp, args.local_rank)
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
    done, t_start, seqs = 0, time.time(), 0
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
            ctx = ddp.no_sync() if not sync else torch.autocast("cpu", enabled=False)
            with ctx, amp:
                loss = crit(ddp(ids, seg, mask), (labels, nsp)) / args.gradient_accumulation_steps
            with (ddp.no_sync() if not sync else torch.autocast("cpu", enabled=False)):
                loss.backward()
            seqs += ids.size(0)
            if not sync:
                continue
            sched.step()
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
    dist.all_reduce(final)
    log.log("summary", training_sequences_per_second=seqs * world / dt, final_loss=float(final) / world,
            ef_buffer_mb=(state.ef_buffer_bytes() / 1e6) if state else 0.0)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
