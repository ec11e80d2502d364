"""Parallel text for the translation driver: two line-aligned files (source, target), a frequency
vocabulary per side, whitespace / punctuation tokenisation.

The reference reads Multi30k through torchtext and spaCy (``examples/MachineTranslation/get_data.py:7-45``:
tokenise, build a vocabulary with ``<unk> <pad> <bos> <eos>`` at indices 0-3, numericalise, pad per
batch).  Neither package nor the data set is available offline, so the same steps are done here on
any pair of aligned text files; ``data.collate_translation`` pads and adds BOS / EOS as before.
"""
from __future__ import annotations

import re
from collections import Counter
from typing import Dict, Iterable, List, Sequence, Tuple

import torch
from torch.utils.data import Dataset

SPECIALS = ("<unk>", "<pad>", "<bos>", "<eos>")
UNK_IDX, PAD_IDX, BOS_IDX, EOS_IDX = 0, 1, 2, 3
_TOKEN = re.compile(r"\w+|[^\w\s]", re.UNICODE)


def tokenize(line: str, lower: bool = True) -> List[str]:
    """Words and single punctuation marks."""
    return _TOKEN.findall(line.lower() if lower else line)


def build_vocab(lines: Iterable[Sequence[str]], min_freq: int = 1, max_size: int = 0) -> Dict[str, int]:
    """Specials first, then tokens by decreasing frequency (ties alphabetical)."""
    counts = Counter(tok for line in lines for tok in line)
    words = sorted((w for w, c in counts.items() if c >= min_freq), key=lambda w: (-counts[w], w))
    if max_size:
        words = words[: max(0, max_size - len(SPECIALS))]
    vocab = {tok: i for i, tok in enumerate(SPECIALS)}
    for w in words:
        vocab.setdefault(w, len(vocab))
    return vocab


class ParallelText(Dataset):
    """``(source ids, target ids)`` tensors without BOS / EOS; lines are paired by position."""

    def __init__(self, src_path: str, tgt_path: str, src_vocab: Dict[str, int] = None,
                 tgt_vocab: Dict[str, int] = None, min_freq: int = 1, max_len: int = 0, lower: bool = True):
        with open(src_path, encoding="utf-8") as f:
            src = [tokenize(line, lower) for line in f]
        with open(tgt_path, encoding="utf-8") as f:
            tgt = [tokenize(line, lower) for line in f]
        if len(src) != len(tgt):
            raise ValueError(f"{src_path} has {len(src)} lines, {tgt_path} has {len(tgt)}")
        pairs = [(s, t) for s, t in zip(src, tgt) if s and t and (not max_len or max(len(s), len(t)) <= max_len)]
        self.src_vocab = src_vocab or build_vocab((s for s, _ in pairs), min_freq)
        self.tgt_vocab = tgt_vocab or build_vocab((t for _, t in pairs), min_freq)
        enc = lambda toks, vocab: torch.tensor([vocab.get(t, UNK_IDX) for t in toks], dtype=torch.long)
        self.pairs: List[Tuple[torch.Tensor, torch.Tensor]] = [(enc(s, self.src_vocab), enc(t, self.tgt_vocab))
                                                               for s, t in pairs]

    def __len__(self):
        return len(self.pairs)

    def __getitem__(self, i):
        return self.pairs[i]

    def decode(self, ids: Sequence[int], side: str = "tgt") -> str:
        vocab = self.tgt_vocab if side == "tgt" else self.src_vocab
        inv = getattr(self, "_inv_" + side, None)
        if inv is None:
            inv = {i: w for w, i in vocab.items()}
            setattr(self, "_inv_" + side, inv)
        return " ".join(inv.get(int(i), "<unk>") for i in ids if int(i) not in (PAD_IDX, BOS_IDX, EOS_IDX))
