"""Workload builders for the benchmark configurations other than the image models.

Each builder returns what ``bench.py`` needs: model, optimizer factory, loss function, a
generator of synthetic host batches of the named shape, samples per step per GPU, the
reducer namespace, the autocast dtype, a description and extra trainer keyword arguments.
All data is synthetic (uniform token ids, random labels) and all weights are random-init.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import models
from .optim import FusedLAMB


def build(args, device, world, ns, gen):
    return {"lstm": _lstm, "transformer": _transformer, "bert": _bert}[args.config](args, device, world, ns, gen)


# ---------------------------------------------------------------------------
def _lstm(args, device, world, ns, gen):
    """3-layer LSTM LM, embedding/hidden 650, tied weights, vocab 33,278, BPTT 35, batch 20 per GPU, fp32;
    RandomBlock hook (10 % blocks) with 8-bit quantised error feedback."""
    vocab, bptt = 33278, 35
    batch = args.batch or 20
    hid, layers = (650, 3) if not args.small else (64, 2)
    model = models.RNNModel("LSTM", vocab, hid, hid, layers, dropout=0.5, tie_weights=True)
    ns.grad_reducer = "conef_randomblock"
    ns.error_compressor = "quant8"
    ns.beta = 0.0            # classic error feedback, stored in 8 bits
    ns.compression_ratio = 0.1

    def forward(ddp, tokens):
        hidden = ddp.module.init_hidden(tokens.size(1))
        out, _ = ddp(tokens, hidden)
        return out

    def make_batch():
        data = torch.randint(0, vocab, (bptt + 1, batch), generator=gen)
        return (data[:-1].contiguous(),), data[1:].reshape(-1).contiguous()

    desc = dict(model="LSTM 3x650 tied, vocab 33278", unit="tok/s", dtype="fp32", seq_len=bptt,
                reducer="RandomBlock 10% + 8-bit quantised error feedback")
    opt = lambda p: torch.optim.SGD(p, lr=1.0)
    return (model, opt, F.nll_loss, make_batch, batch * bptt, ns, None, desc,
            dict(forward_fn=forward, grad_clip=0.25))


# ---------------------------------------------------------------------------
def _transformer(args, device, world, ns, gen):
    """Transformer-base encoder-decoder (6+6, d 512, 8 heads, FFN 2048, shared vocab 32,000), bf16,
    about 4,096 tokens per GPU with source / target lengths uniform in [10, 100];
    hPowerSGD rank 8 with low-rank compressed error feedback."""
    vocab = 32000
    sentences = args.batch or 37             # 37 * (55 + 55) average tokens = 4,070
    if args.small:
        model = models.Seq2SeqTransformer(2, 2, 64, 4, vocab, vocab, 128, 0.1)
    else:
        model = models.Seq2SeqTransformer(6, 6, 512, 8, vocab, vocab, 2048, 0.1)
    model.tgt_tok_emb.embedding.weight = model.src_tok_emb.embedding.weight      # shared vocabulary
    ns.grad_reducer = "hefsgd_powersgd"
    ns.error_compressor = "lowrank"
    ns.matrix_approximation_rank = 8
    ns.error_rank = 8
    pad = models.seq2seq.PAD_IDX

    def make_batch():
        src_len = torch.randint(10, 101, (sentences,), generator=gen)
        tgt_len = torch.randint(10, 101, (sentences,), generator=gen)
        src = torch.full((101, sentences), pad, dtype=torch.long)
        tgt = torch.full((102, sentences), pad, dtype=torch.long)
        for i in range(sentences):
            src[: src_len[i], i] = torch.randint(4, vocab, (int(src_len[i]),), generator=gen)
            tgt[: tgt_len[i] + 1, i] = torch.randint(4, vocab, (int(tgt_len[i]) + 1,), generator=gen)
        return (src, tgt[:-1].contiguous()), tgt[1:].contiguous()

    def forward(ddp, src, tgt_in):
        sm, tm, sp, tp = models.seq2seq.create_mask(src, tgt_in, pad)
        return ddp(src, tgt_in, sm, tm, sp, tp, sp)

    def loss_fn(logits, tgt_out):
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), tgt_out.reshape(-1), ignore_index=pad)

    desc = dict(model="Transformer-base 6+6 (shared vocab 32000)", unit="tok/s", dtype="bf16", seq_len=101,
                reducer="hPowerSGD rank 8 + low-rank (rank 8) error feedback")
    opt = lambda p: torch.optim.Adam(p, lr=1e-4, betas=(0.9, 0.98), eps=1e-9)
    tokens_per_step = sentences * 110          # expected source + target tokens (lengths uniform in [10, 100])
    return model, opt, loss_fn, make_batch, tokens_per_step, ns, torch.bfloat16, desc, dict(forward_fn=forward)


# ---------------------------------------------------------------------------
def _bert(args, device, world, ns, gen):
    """BERT-large pre-training (24 layers, hidden 1024, 16 heads, FFN 4096, vocab 30,522 padded to 30,528),
    bf16, sequence 128, batch 64 per GPU, 15 % MLM masking, random NSP labels, LAMB;
    PowerSGD rank 8 with ConEF count-sketch error compression."""
    seq = 128
    batch = args.batch or 64
    if args.small:
        cfg = models.BertConfig(30528, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                intermediate_size=256)
    else:
        cfg = models.BertConfig.large(30528)
    model = models.BertForPreTraining(cfg)
    ns.grad_reducer = "conef_powersgd"
    ns.matrix_approximation_rank = 8
    ns.sketch_size = 0.1
    crit = models.BertPretrainingCriterion(cfg.vocab_size)

    def make_batch():
        ids = torch.randint(1000, 30522, (batch, seq), generator=gen)
        seg = torch.zeros(batch, seq, dtype=torch.long)
        seg[:, seq // 2 :] = 1
        mask = torch.ones(batch, seq, dtype=torch.long)
        labels = torch.full((batch, seq), -1, dtype=torch.long)
        chosen = torch.rand(batch, seq, generator=gen) < 0.15
        labels[chosen] = ids[chosen]
        ids = ids.clone()
        ids[chosen] = 103                                    # [MASK]
        nsp = torch.randint(0, 2, (batch,), generator=gen)
        return (ids, seg, mask), (labels, nsp)

    def opt(params):
        params = list(params)
        decay = [p for p in params if p.dim() > 1]
        no_decay = [p for p in params if p.dim() <= 1]
        return FusedLAMB([{"params": decay, "weight_decay": 0.01}, {"params": no_decay, "weight_decay": 0.0}],
                         lr=1.25e-3)

    desc = dict(model="BERT-large (vocab 30528)" if not args.small else "BERT-tiny (smoke)", unit="seq/s",
                dtype="bf16", seq_len=seq, reducer="PowerSGD rank 8 + ConEF count sketch 10%, beta 0.9")
    return model, opt, crit, make_batch, batch, ns, torch.bfloat16, desc, {}
