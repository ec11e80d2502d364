#!/usr/bin/env python
"""Word-level language modelling (LSTM / GRU / RNN / Transformer) with compressed gradients.

Counterpart of the reference's ``examples/LanguageModeling/main.py``: global batch cut into
per-rank columns, truncated BPTT with hidden-state repackaging, ``clip_grad_norm_(0.25)`` after
the hook has run, SGD or Adam, validation perplexity per epoch.  ``--data`` points at a directory
with ``train.txt / valid.txt / test.txt``; without it a synthetic token stream is used.
"""
import argparse
import math
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import conef_b200 as cb  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.data import Corpus, batchify, get_batch, synthetic_token_stream  # noqa: E402
from conef_b200.utils import GracefulStop, JsonLogger  # noqa: E402


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--data", default=None)
    p.add_argument("--model", default="LSTM", help="LSTM, GRU, RNN_TANH, RNN_RELU or Transformer")
    p.add_argument("--emsize", type=int, default=672)
    p.add_argument("--nhid", type=int, default=672)
    p.add_argument("--nlayers", type=int, default=2)
    p.add_argument("--nhead", type=int, default=2)
    p.add_argument("--lr", type=float, default=20)
    p.add_argument("--optimizer", default="sgd", choices=["sgd", "adam"])
    p.add_argument("--clip", type=float, default=0.25)
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--batch_size", type=int, default=20, help="per process")
    p.add_argument("--bptt", type=int, default=35)
    p.add_argument("--dropout", type=float, default=0.2)
    p.add_argument("--tied", action="store_true")
    p.add_argument("--vocab", type=int, default=33278, help="synthetic data only")
    p.add_argument("--tokens", type=int, default=200_000, help="synthetic data only")
    p.add_argument("--grad_reducer", default="conef_randomblock", choices=cb.REDUCERS)
    p.add_argument("--start_compression_iter", type=int, default=10)
    p.add_argument("--compression_ratio", type=float, default=0.1)
    p.add_argument("--beta", type=float, default=0.9)
    p.add_argument("--sketch_size", type=float, default=0.2)
    p.add_argument("--matrix_approximation_rank", type=int, default=4)
    p.add_argument("--min_compression_rate", type=float, default=2)
    p.add_argument("--orthogonalization_epsilon", type=float, default=0)
    p.add_argument("--error_compressor", default=None)
    p.add_argument("--seed", type=int, default=1111)
    return p.parse_args()


def evaluate(net, data, bptt, ntokens, is_transformer, device):
    net.eval()
    total, crit = 0.0, nn.NLLLoss()
    hidden = None if is_transformer else net.init_hidden(data.size(1))
    with torch.no_grad():
        for i in range(0, data.size(0) - 1, bptt):
            x, y = get_batch(data, i, bptt)
            x, y = x.to(device), y.to(device)
            if is_transformer:
                out = net(x).view(-1, ntokens)
            else:
                out, hidden = net(x, hidden)
                hidden = models.repackage_hidden(hidden)
            total += len(x) * float(crit(out, y))
    return total / max(1, data.size(0) - 1)


def main():
    args = parse()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29502")
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    torch.manual_seed(args.seed)
    if args.data:
        corpus = Corpus(args.data)
        ntokens, train, valid = len(corpus.dictionary), corpus.train, corpus.valid
    else:
        ntokens = args.vocab
        train = synthetic_token_stream(args.tokens, ntokens, 0)
        valid = synthetic_token_stream(args.tokens // 10, ntokens, 1)
    train = batchify(train, args.batch_size * world, rank, world)
    valid = batchify(valid, 10, 0, 1)
    is_tf = args.model == "Transformer"
    net = (models.TransformerModel(ntokens, args.emsize, args.nhead, args.nhid, args.nlayers, args.dropout) if is_tf
           else models.RNNModel(args.model, ntokens, args.emsize, args.nhid, args.nlayers, args.dropout, args.tied))
    net = net.to(device)
    ddp = DDP(net, device_ids=[local] if cuda else None, gradient_as_bucket_view=True)
    state = cb.get_comm_hooks(args, ddp, local)
    opt = (torch.optim.SGD(ddp.parameters(), lr=args.lr) if args.optimizer == "sgd"
           else torch.optim.Adam(ddp.parameters(), lr=args.lr))
    crit, stop, log = nn.NLLLoss(), GracefulStop(), JsonLogger()
    for epoch in range(args.epochs):
        ddp.train()
        hidden = None if is_tf else net.init_hidden(args.batch_size)
        t0, tokens = time.time(), 0
        for i in range(0, train.size(0) - 1, args.bptt):
            x, y = get_batch(train, i, args.bptt)
            x, y = x.to(device, non_blocking=True), y.to(device, non_blocking=True)
            opt.zero_grad(set_to_none=False)
            if is_tf:
                out = ddp(x).view(-1, ntokens)
            else:
                hidden = models.repackage_hidden(hidden)      # truncated BPTT
                out, hidden = ddp(x, hidden)
            loss = crit(out, y)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(ddp.parameters(), args.clip)   # after the hook, as the reference
            opt.step()
            tokens += y.numel()
            if stop.requested:
                break
        val = evaluate(net, valid, args.bptt, ntokens, is_tf, device)
        log.log(epoch, train_loss=float(loss), valid_loss=val, valid_ppl=math.exp(min(val, 20)),
                tok_per_s=tokens * world / (time.time() - t0),
                ef_buffer_mb=(state.ef_buffer_bytes() / 1e6) if state else 0.0)
        if stop.requested:
            break
    if state is not None:
        state.check_status()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
