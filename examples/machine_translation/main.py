#!/usr/bin/env python
"""Transformer encoder-decoder translation with compressed gradients.

Counterpart of the reference's ``examples/MachineTranslation/{main,train_n_test}.py``:
``Seq2SeqTransformer`` (default 3+3 layers, d 512, FFN 512), Adam(0.9, 0.98, 1e-9), a global
batch of sentence pairs sliced per rank, padding / causal masks, validation loss per epoch.
The reference reads Multi30k through torchtext + spacy, neither of which is installed here;
sentence pairs are synthetic (lengths uniform in [10, 100], uniform token ids).
"""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import conef_b200 as cb  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.data import ParallelText, SyntheticTranslationPairs, collate_translation  # noqa: E402
from conef_b200.utils import GracefulStop, JsonLogger  # noqa: E402

PAD = models.seq2seq.PAD_IDX


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--pairs", type=int, default=2000, help="synthetic sentence pairs per epoch")
    p.add_argument("--train_src", default=None, help="source-language text, one sentence per line (with --train_tgt: "
                                                    "train on these files instead of synthetic pairs)")
    p.add_argument("--train_tgt", default=None)
    p.add_argument("--valid_src", default=None)
    p.add_argument("--valid_tgt", default=None)
    p.add_argument("--min_freq", type=int, default=1)
    p.add_argument("--max_len", type=int, default=100)
    p.add_argument("--batch_size", type=int, default=32, help="sentence pairs per process")
    p.add_argument("--vocab", type=int, default=32000)
    p.add_argument("--num_encoder_layers", type=int, default=3)
    p.add_argument("--num_decoder_layers", type=int, default=3)
    p.add_argument("--emb_size", type=int, default=512)
    p.add_argument("--nhead", type=int, default=8)
    p.add_argument("--ffn_hid_dim", type=int, default=512)
    p.add_argument("--dropout", type=float, default=0.1)
    p.add_argument("--lr", type=float, default=1e-4)
    p.add_argument("--bf16", action="store_true")
    p.add_argument("--grad_reducer", default="hefsgd_powersgd", choices=cb.REDUCERS)
    p.add_argument("--start_compression_iter", type=int, default=10)
    p.add_argument("--compression_ratio", type=float, default=0.1)
    p.add_argument("--beta", type=float, default=0.9)
    p.add_argument("--sketch_size", type=float, default=0.2)
    p.add_argument("--matrix_approximation_rank", type=int, default=8)
    p.add_argument("--min_compression_rate", type=float, default=2)
    p.add_argument("--orthogonalization_epsilon", type=float, default=0)
    p.add_argument("--error_compressor", default=None)
    p.add_argument("--error_rank", type=int, default=None)
    p.add_argument("--seed", type=int, default=0)
    return p.parse_args()


def forward(ddp, src, tgt_in):
    sm, tm, sp, tp = models.create_mask(src, tgt_in, PAD)
    return ddp(src, tgt_in, sm, tm, sp, tp, sp)


def loss_fn(logits, tgt_out):
    return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), tgt_out.reshape(-1), ignore_index=PAD)


def main():
    args = parse()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29503")
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    torch.manual_seed(args.seed)
    if args.train_src and args.train_tgt:
        train = ParallelText(args.train_src, args.train_tgt, min_freq=args.min_freq, max_len=args.max_len)
        valid = ParallelText(args.valid_src, args.valid_tgt, train.src_vocab, train.tgt_vocab, max_len=args.max_len) \
            if (args.valid_src and args.valid_tgt) else train
        src_vocab, tgt_vocab = len(train.src_vocab), len(train.tgt_vocab)
    else:
        train = SyntheticTranslationPairs(args.pairs, args.vocab, args.vocab, seed=1)
        valid = SyntheticTranslationPairs(max(64, args.pairs // 10), args.vocab, args.vocab, seed=2)
        src_vocab = tgt_vocab = args.vocab
    net = models.Seq2SeqTransformer(args.num_encoder_layers, args.num_decoder_layers, args.emb_size, args.nhead,
                                    src_vocab, tgt_vocab, args.ffn_hid_dim, args.dropout)
    for p in net.parameters():
        if p.dim() > 1:
            torch.nn.init.xavier_uniform_(p)
    trainer = cb.DataParallelTrainer(
        net, lambda p: torch.optim.Adam(p, lr=args.lr, betas=(0.9, 0.98), eps=1e-9), loss_fn, reducer=args,
        device=device, autocast_dtype=torch.bfloat16 if (args.bf16 and cuda) else None, forward_fn=forward)
    sampler = DistributedSampler(train, world, rank, shuffle=True, seed=args.seed)
    loader = DataLoader(train, args.batch_size, sampler=sampler, collate_fn=collate_translation, drop_last=True)
    vloader = DataLoader(valid, args.batch_size, collate_fn=collate_translation)
    stop, log = GracefulStop(), JsonLogger()
    for epoch in range(args.epochs):
        sampler.set_epoch(epoch)
        trainer.model.train()
        t0, tokens, total = time.time(), 0, 0.0
        for src, tgt in loader:
            loss = trainer.step((src, tgt[:-1].contiguous()), tgt[1:].contiguous())
            total += float(loss)
            tokens += int((src != PAD).sum() + (tgt[1:] != PAD).sum())
            if stop.requested:
                break
        trainer.model.eval()
        vloss, n = 0.0, 0
        with torch.no_grad():
            for src, tgt in vloader:
                src, tgt = src.to(device), tgt.to(device)
                vloss += float(loss_fn(forward(trainer.model, src, tgt[:-1]), tgt[1:]))
                n += 1
        log.log(epoch, train_loss=total / max(1, len(loader)), valid_loss=vloss / max(1, n),
                tok_per_s=tokens * world / (time.time() - t0),
                ef_buffer_mb=(trainer.state.ef_buffer_bytes() / 1e6) if trainer.state else 0.0)
        if stop.requested:
            break
    trainer.check()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
