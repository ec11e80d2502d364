"""Word-level corpus and batching for the language-model example.

``Dictionary`` / ``Corpus`` read ``train.txt`` / ``valid.txt`` / ``test.txt`` from a directory
when it exists (format of the reference's ``examples/LanguageModeling/data.py:20-48``:
whitespace tokens plus ``<eos>`` per line); ``batchify`` and ``get_batch`` shape the token
stream as in ``main.py:69-85,137-144``: a global batch is cut from the stream and every rank
takes its own columns.
"""
from __future__ import annotations

import os

import torch


class Dictionary:
    def __init__(self):
        self.word2idx, self.idx2word = {}, []

    def add_word(self, word):
        if word not in self.word2idx:
            self.idx2word.append(word)
            self.word2idx[word] = len(self.idx2word) - 1
        return self.word2idx[word]

    def __len__(self):
        return len(self.idx2word)


class Corpus:
    def __init__(self, path):
        self.dictionary = Dictionary()
        self.train = self.tokenize(os.path.join(path, "train.txt"))
        self.valid = self.tokenize(os.path.join(path, "valid.txt"))
        self.test = self.tokenize(os.path.join(path, "test.txt"))

    def tokenize(self, path):
        assert os.path.exists(path), path
        ids = []
        with open(path, "r", encoding="utf8") as fh:
            for line in fh:
                ids.extend(self.dictionary.add_word(w) for w in line.split() + ["<eos>"])
        return torch.tensor(ids, dtype=torch.int64)


def batchify(data: torch.Tensor, global_batch: int, rank: int = 0, world: int = 1) -> torch.Tensor:
    """Stream -> ``(steps, global_batch)`` columns, then this rank's ``global_batch / world`` columns."""
    nbatch = data.size(0) // global_batch
    data = data[: nbatch * global_batch].view(global_batch, -1).t().contiguous()
    per = global_batch // world
    return data[:, rank * per : (rank + 1) * per].contiguous()


def get_batch(source: torch.Tensor, i: int, bptt: int):
    seq_len = min(bptt, len(source) - 1 - i)
    return source[i : i + seq_len], source[i + 1 : i + 1 + seq_len].reshape(-1)
