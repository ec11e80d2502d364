"""Shared plumbing of the fine-tuning drivers (``run_glue.py``, ``run_squad.py``, ``run_swag.py``):
arguments, process group, model configuration, checkpoint loading and the training loop.

Every driver trains under DistributedDataParallel with the reducer named by ``--grad_reducer`` (the
hooks of ``conef_b200.get_comm_hooks``; plain all-reduce by default, since fine-tuning runs are short),
BertAdam with linear warm-up, optional gradient accumulation (``no_sync`` on all but the last
micro-batch) and bf16 autocast.  A driver supplies the model, the number of training items and a
function that maps a tensor of item indices to a loss.
"""
import argparse
import os
import sys
import time
from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import conef_b200 as cb  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.optim import BertAdam  # noqa: E402


def add_common_arguments(p: argparse.ArgumentParser, *, batch: int, lr: float, epochs: float, seed: int,
                         max_seq_length: int) -> None:
    p.add_argument("--vocab_file", required=True)
    p.add_argument("--bert_model", default="large", choices=["large", "base", "tiny"])
    p.add_argument("--config_file", default=None)
    p.add_argument("--init_checkpoint", default=None,
                   help="pre-training or fine-tuned checkpoint ('model' state dict); random weights without")
    p.add_argument("--do_lower_case", action="store_true", default=True)
    p.add_argument("--max_seq_length", type=int, default=max_seq_length)
    p.add_argument("--train_batch_size", type=int, default=batch, help="items per process and optimizer step")
    p.add_argument("--gradient_accumulation_steps", type=int, default=1)
    p.add_argument("--learning_rate", type=float, default=lr)
    p.add_argument("--warmup_proportion", type=float, default=0.1)
    p.add_argument("--num_train_epochs", type=float, default=epochs)
    p.add_argument("--max_steps", type=int, default=-1, help="stop after this many optimizer steps when positive")
    p.add_argument("--bf16", action="store_true")
    p.add_argument("--no_cuda", action="store_true")
    p.add_argument("--seed", type=int, default=seed)
    p.add_argument("--grad_reducer", default="allreduce", choices=cb.REDUCERS)
    p.add_argument("--start_compression_percentage", type=float, default=0.1)
    p.add_argument("--compression_ratio", type=float, default=0.1)
    p.add_argument("--sketch_size", type=float, default=0.1)
    p.add_argument("--beta", type=float, default=0.9)
    p.add_argument("--matrix_approximation_rank", type=int, default=8)
    p.add_argument("--min_compression_rate", type=float, default=2)
    p.add_argument("--orthogonalization_epsilon", type=float, default=0)
    p.add_argument("--error_compressor", default=None)
    p.add_argument("--local_rank", type=int, default=int(os.environ.get("LOCAL_RANK", 0)))


def check_common_arguments(p: argparse.ArgumentParser, args) -> None:
    if args.gradient_accumulation_steps < 1 or args.train_batch_size % args.gradient_accumulation_steps:
        p.error("--train_batch_size must be a positive multiple of --gradient_accumulation_steps")


@dataclass
class Runtime:
    rank: int
    world: int
    device: torch.device
    cuda: bool
    use_ddp: bool
    own_group: bool
    amp: Callable

    def tensor(self, rows, dtype=torch.long):
        return torch.tensor(rows, dtype=dtype, device=self.device)


def init_runtime(args, training: bool, port: str) -> Runtime:
    """Device, autocast context and (for training on several ranks or with a compression hook) the
    process group; a group this function creates is destroyed again by ``finish``."""
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    cuda = torch.cuda.is_available() and not args.no_cuda
    device = torch.device("cuda", max(args.local_rank, 0)) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    use_ddp = training and (world > 1 or args.grad_reducer != "allreduce")
    own_group = False
    if (use_ddp or world > 1) and not dist.is_initialized():      # several ranks also share evaluation work
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", port)
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
        own_group = True
    torch.manual_seed(args.seed)
    amp = (lambda: torch.autocast("cuda", dtype=torch.bfloat16)) if (args.bf16 and cuda) \
        else (lambda: torch.autocast("cpu", enabled=False))
    return Runtime(rank, world, device, cuda, use_ddp, own_group, amp)


def finish(rt: Runtime) -> None:
    if dist.is_initialized():
        dist.barrier()
        if rt.own_group:
            dist.destroy_process_group()


def bert_config(args, vocab_size: int):
    if args.config_file:
        cfg = models.BertConfig.from_json_file(args.config_file)
    elif args.bert_model == "large":
        cfg = models.BertConfig.large()
    elif args.bert_model == "base":
        cfg = models.BertConfig.base()
    else:
        cfg = models.BertConfig(max(vocab_size, 8), hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                intermediate_size=512)
    if cfg.vocab_size % 8 != 0:                 # pre-training pads the vocabulary to a multiple of 8
        cfg.vocab_size += 8 - cfg.vocab_size % 8
    return cfg


def load_matching_weights(net, path):
    """Take every tensor of the checkpoint whose name and shape match (a pre-training checkpoint has the
    encoder but not the task head; a fine-tuned one has both); returns the names left at their
    initial values."""
    blob = torch.load(path, map_location="cpu", weights_only=False)
    sd = blob.get("model", blob)
    own = net.state_dict()
    take = {k: v for k, v in sd.items() if k in own and tuple(v.shape) == tuple(own[k].shape)}
    net.load_state_dict(take, strict=False)
    return sorted(set(own) - set(take))


class _NoContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def train(net, args, rt: Runtime, n_items: int, loss_of: Callable) -> dict:
    """The training loop.  ``loss_of(model, index)`` returns the mean loss of the items ``index`` (a
    long tensor on the device).  Every rank takes the same number of items per epoch from one seeded
    permutation, so all ranks run the same number of steps."""
    per_rank = n_items // rt.world
    steps_per_epoch = max(per_rank // args.train_batch_size, 1)
    total = int(steps_per_epoch * args.num_train_epochs)
    if args.max_steps > 0:
        total = min(total, args.max_steps)
    total = max(total, 1)
    args.start_compression_iter = max(2, int(total * args.start_compression_percentage))
    decay = [p for n, p in net.named_parameters() if p.requires_grad and p.dim() > 1]
    no_decay = [p for n, p in net.named_parameters() if p.requires_grad and p.dim() <= 1]
    opt = BertAdam([{"params": decay, "weight_decay": 0.01}, {"params": no_decay, "weight_decay": 0.0}],
                   lr=args.learning_rate, warmup=args.warmup_proportion, t_total=total)
    model, state = net, None
    if rt.use_ddp:
        model = DDP(net, device_ids=[rt.device.index] if rt.cuda else None, gradient_as_bucket_view=True)
        state = cb.get_comm_hooks(args, model, args.local_rank)
    micro = args.train_batch_size // args.gradient_accumulation_steps
    step, t0, losses = 0, time.time(), []
    while step < total:
        epoch = step // steps_per_epoch
        g = torch.Generator().manual_seed(args.seed + epoch)          # same permutation on every rank
        order = torch.randperm(n_items, generator=g)[rt.rank::rt.world][:per_rank].to(rt.device)
        for b in range(steps_per_epoch):
            if step >= total:
                break
            net.train()
            idx = order[b * args.train_batch_size:(b + 1) * args.train_batch_size]
            opt.zero_grad(set_to_none=True)
            loss_value = 0.0
            for a in range(args.gradient_accumulation_steps):
                part = idx[a * micro:(a + 1) * micro]
                if part.numel() == 0:
                    continue
                last = a == args.gradient_accumulation_steps - 1
                sync = model.no_sync if (rt.use_ddp and not last) else _NoContext
                with sync(), rt.amp():
                    loss = loss_of(model, part) / args.gradient_accumulation_steps
                loss.backward()
                loss_value += float(loss.detach())
            opt.step()
            losses.append(loss_value)
            step += 1
    if state is not None and hasattr(state, "check_status"):
        state.check_status()
    return {"train_steps": step, "train_loss_first": losses[0],
            "train_loss_last": sum(losses[-10:]) / len(losses[-10:]),      # mean of the last ten steps
            "train_seq_per_s": step * args.train_batch_size * rt.world / max(time.time() - t0, 1e-9)}
