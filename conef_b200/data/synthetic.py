"""Synthetic datasets of the benchmark shapes (there is no network for real corpora).

Each dataset is an ordinary ``torch.utils.data.Dataset`` with deterministic content so
that ``DistributedSampler`` / rank slicing behave as with real data.
"""
from __future__ import annotations

import torch
from torch.utils.data import Dataset


class SyntheticImages(Dataset):
    """N(0,1) images of shape ``(3, size, size)`` with uniform labels (CIFAR-shaped by default)."""

    def __init__(self, length=50_000, num_classes=10, size=32, seed=0):
        self.length, self.num_classes, self.size, self.seed = length, num_classes, size, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        return torch.randn(3, self.size, self.size, generator=g), int(torch.randint(0, self.num_classes, (1,), generator=g))


def synthetic_token_stream(num_tokens: int, vocab: int, seed: int = 0) -> torch.Tensor:
    """A flat stream of uniform token ids (WikiText-shaped language-model data)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (num_tokens,), generator=g)


class SyntheticTranslationPairs(Dataset):
    """Sentence pairs with lengths uniform in ``[lo, hi]`` and uniform token ids (ids < 4 are specials)."""

    def __init__(self, length=29_000, src_vocab=32_000, tgt_vocab=32_000, lo=10, hi=100, seed=0):
        self.length, self.src_vocab, self.tgt_vocab, self.lo, self.hi, self.seed = length, src_vocab, tgt_vocab, lo, hi, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        ls, lt = (int(torch.randint(self.lo, self.hi + 1, (1,), generator=g)) for _ in range(2))
        return (torch.randint(4, self.src_vocab, (ls,), generator=g), torch.randint(4, self.tgt_vocab, (lt,), generator=g))


def collate_translation(batch, pad_idx=1, bos_idx=2, eos_idx=3):
    """Sequence-first padded batches with BOS / EOS, as the reference's ``get_data.py:27-45``."""
    def pack(seqs):
        full = [torch.cat([torch.tensor([bos_idx]), s, torch.tensor([eos_idx])]) for s in seqs]
        return torch.nn.utils.rnn.pad_sequence(full, padding_value=pad_idx)
    return pack([b[0] for b in batch]), pack([b[1] for b in batch])


class SyntheticBertShard(Dataset):
    """Pre-training instances in the reference's HDF5 field layout
    (``input_ids, segment_ids, input_mask, masked_lm_labels, next_sentence_labels``;
    ``run_pretraining_conef.py:102-131``), generated instead of read from disk."""

    def __init__(self, length=4096, seq_len=128, vocab=30522, max_pred=20, seed=0):
        self.length, self.seq_len, self.vocab, self.max_pred, self.seed = length, seq_len, vocab, max_pred, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        from .masking import mask_tokens

        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        ids = torch.randint(1000, self.vocab, (self.seq_len,), generator=g)
        ids[0], ids[self.seq_len // 2], ids[-1] = 101, 102, 102          # [CLS] A [SEP] B [SEP]
        seg = torch.zeros(self.seq_len, dtype=torch.long)
        seg[self.seq_len // 2 + 1 :] = 1
        masked, labels = mask_tokens(ids, self.vocab, 0.15, self.max_pred, g)
        nsp = int(torch.randint(0, 2, (1,), generator=g))
        return masked, seg, torch.ones(self.seq_len, dtype=torch.long), labels, nsp
