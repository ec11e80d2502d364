"""BERT pre-training data: documents -> (sentence pair, masked LM) instances -> shard files ->
dataset with the next shard loaded in the background.

The reference does this with ``create_pretraining_data.py`` (instances from tokenised documents
``:219-312``, masking ``:314-364``, HDF5 writer ``:65-142``), an HDF5 dataset
(``run_pretraining_conef.py:102-131``) and a one-worker process pool that opens the next shard
while the current one trains (``:567-754``).  Here the shard container is a NumPy ``.npz`` archive
with the same six fields (``input_ids, input_mask, segment_ids, masked_lm_positions,
masked_lm_ids, next_sentence_labels``); nothing else about the recipe changes.
"""
from __future__ import annotations

import glob
import os
import random
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass
from typing import Iterable, Iterator, List, Optional, Sequence

import numpy as np
import torch
from torch.utils.data import Dataset

FIELDS = ("input_ids", "input_mask", "segment_ids", "masked_lm_positions", "masked_lm_ids",
          "next_sentence_labels")


@dataclass
class TrainingInstance:
    tokens: List[str]
    segment_ids: List[int]
    is_random_next: bool
    masked_lm_positions: List[int]
    masked_lm_labels: List[str]


def read_documents(paths: Iterable[str], tokenizer) -> List[List[List[str]]]:
    """One sentence per line, documents separated by blank lines -> ``[document][sentence][token]``."""
    docs: List[List[List[str]]] = [[]]
    for path in paths:
        with open(path, encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if not line:
                    if docs[-1]:
                        docs.append([])
                    continue
                toks = tokenizer.tokenize(line)
                if toks:
                    docs[-1].append(toks)
        if docs[-1]:
            docs.append([])
    return [d for d in docs if d]


def _truncate_pair(a: List[str], b: List[str], max_tokens: int, rng: random.Random) -> None:
    while len(a) + len(b) > max_tokens:
        longer = a if len(a) > len(b) else b
        if rng.random() < 0.5:
            del longer[0]
        else:
            longer.pop()


def create_masked_lm_predictions(tokens: List[str], masked_lm_prob: float, max_predictions: int,
                                 vocab_words: Sequence[str], rng: random.Random):
    """15 % of the positions (never [CLS]/[SEP]) are predicted: 80 % become [MASK], 10 % a random
    word, 10 % stay."""
    cand = [i for i, t in enumerate(tokens) if t not in ("[CLS]", "[SEP]")]
    rng.shuffle(cand)
    n_pred = min(max_predictions, max(1, int(round(len(tokens) * masked_lm_prob))))
    out = list(tokens)
    picked = sorted(cand[:n_pred])
    labels = []
    for i in picked:
        roll = rng.random()
        if roll < 0.8:
            out[i] = "[MASK]"
        elif roll < 0.9:
            out[i] = vocab_words[rng.randint(0, len(vocab_words) - 1)]
        labels.append(tokens[i])
    return out, picked, labels


def create_instances_from_document(docs, index: int, max_seq_length: int, short_seq_prob: float,
                                   masked_lm_prob: float, max_predictions: int, vocab_words, rng) -> List[TrainingInstance]:
    """Sentence-pair instances of one document: segment A is a run of its sentences, segment B either
    continues the document or (half of the time, and always for one-chunk documents) comes from a
    random other document; unused sentences are put back."""
    doc = docs[index]
    max_tokens = max_seq_length - 3
    target = rng.randint(2, max_tokens) if rng.random() < short_seq_prob else max_tokens
    out, chunk, length, i = [], [], 0, 0
    while i < len(doc):
        chunk.append(doc[i])
        length += len(doc[i])
        if i == len(doc) - 1 or length >= target:
            if chunk:
                a_end = rng.randint(1, len(chunk) - 1) if len(chunk) >= 2 else 1
                a = [t for s in chunk[:a_end] for t in s]
                b: List[str] = []
                random_next = len(chunk) == 1 or rng.random() < 0.5
                if random_next and len(docs) > 1:
                    for _ in range(10):
                        other = rng.randint(0, len(docs) - 1)
                        if other != index:
                            break
                    rdoc = docs[other]
                    start = rng.randint(0, len(rdoc) - 1)
                    for s in rdoc[start:]:
                        b.extend(s)
                        if len(b) >= target - len(a):
                            break
                    i -= len(chunk) - a_end            # put the unused sentences back
                else:
                    random_next = False
                    b = [t for s in chunk[a_end:] for t in s]
                if not b:                              # single-document corpus with a one-sentence chunk
                    half = max(1, len(a) // 2)
                    a, b = a[:half], a[half:] or a[:1]
                _truncate_pair(a, b, max_tokens, rng)
                tokens = ["[CLS]"] + a + ["[SEP]"] + b + ["[SEP]"]
                seg = [0] * (len(a) + 2) + [1] * (len(b) + 1)
                masked, pos, labels = create_masked_lm_predictions(tokens, masked_lm_prob, max_predictions,
                                                                   vocab_words, rng)
                out.append(TrainingInstance(masked, seg, random_next, pos, labels))
            chunk, length = [], 0
        i += 1
    return out


def create_training_instances(docs, vocab_words, max_seq_length=128, dupe_factor=5, short_seq_prob=0.1,
                              masked_lm_prob=0.15, max_predictions_per_seq=20, seed=12345) -> List[TrainingInstance]:
    rng = random.Random(seed)
    docs = list(docs)
    rng.shuffle(docs)
    # random replacements never introduce a control token such as [SEP] or [PAD]
    vocab_words = [w for w in vocab_words if not (w.startswith("[") and w.endswith("]"))]
    out: List[TrainingInstance] = []
    for _ in range(dupe_factor):
        for k in range(len(docs)):
            out.extend(create_instances_from_document(docs, k, max_seq_length, short_seq_prob, masked_lm_prob,
                                                      max_predictions_per_seq, vocab_words, rng))
    rng.shuffle(out)
    return out


def instances_to_arrays(instances: Sequence[TrainingInstance], tokenizer, max_seq_length: int,
                        max_predictions_per_seq: int) -> dict:
    n = len(instances)
    arr = {"input_ids": np.zeros((n, max_seq_length), np.int32),
           "input_mask": np.zeros((n, max_seq_length), np.int8),
           "segment_ids": np.zeros((n, max_seq_length), np.int8),
           "masked_lm_positions": np.zeros((n, max_predictions_per_seq), np.int32),
           "masked_lm_ids": np.zeros((n, max_predictions_per_seq), np.int32),
           "next_sentence_labels": np.zeros((n,), np.int8)}
    for k, inst in enumerate(instances):
        ids = tokenizer.convert_tokens_to_ids(inst.tokens)
        L = len(ids)
        arr["input_ids"][k, :L] = ids
        arr["input_mask"][k, :L] = 1
        arr["segment_ids"][k, :L] = inst.segment_ids
        P = len(inst.masked_lm_positions)
        arr["masked_lm_positions"][k, :P] = inst.masked_lm_positions
        arr["masked_lm_ids"][k, :P] = tokenizer.convert_tokens_to_ids(inst.masked_lm_labels)
        arr["next_sentence_labels"][k] = int(inst.is_random_next)
    return arr


def write_shard(path: str, arrays: dict) -> None:
    missing = [f for f in FIELDS if f not in arrays]
    if missing:
        raise ValueError(f"shard is missing fields {missing}")
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        np.savez_compressed(f, **{k: arrays[k] for k in FIELDS})
    os.replace(tmp, path)


def load_shard(path: str) -> dict:
    with np.load(path) as z:
        return {k: z[k] for k in FIELDS}


class PretrainingShard(Dataset):
    """One shard as a dataset of ``(input_ids, segment_ids, input_mask, masked_lm_labels,
    next_sentence_labels)``; the dense label row holds ``-1`` where nothing is predicted (padded
    prediction slots have position 0 and are dropped)."""

    def __init__(self, arrays_or_path, max_pred_length: Optional[int] = None):
        self.arrays = load_shard(arrays_or_path) if isinstance(arrays_or_path, (str, os.PathLike)) else arrays_or_path
        self.max_pred_length = max_pred_length or self.arrays["masked_lm_positions"].shape[1]

    def __len__(self):
        return len(self.arrays["input_ids"])

    def __getitem__(self, i):
        a = self.arrays
        ids = torch.from_numpy(a["input_ids"][i].astype(np.int64))
        mask = torch.from_numpy(a["input_mask"][i].astype(np.int64))
        seg = torch.from_numpy(a["segment_ids"][i].astype(np.int64))
        pos = a["masked_lm_positions"][i][: self.max_pred_length]
        lab = a["masked_lm_ids"][i][: self.max_pred_length]
        n = int((pos != 0).sum())                 # position 0 is [CLS]: never predicted, so 0 means padding
        labels = torch.full_like(ids, -1)
        if n:
            labels[torch.from_numpy(pos[:n].astype(np.int64))] = torch.from_numpy(lab[:n].astype(np.int64))
        return ids, seg, mask, labels, int(a["next_sentence_labels"][i])


def shard_files(input_dir: str, rank: int = 0, world: int = 1, epoch: int = 0, seed: int = 0) -> List[str]:
    """This rank's shard files for an epoch: all ranks shuffle with the same seed and take every
    ``world``-th file, starting at their rank (wrapping when there are fewer files than ranks)."""
    files = sorted(glob.glob(os.path.join(input_dir, "*.npz")))
    if not files:
        raise FileNotFoundError(f"no .npz shards under {input_dir}")
    random.Random(seed + epoch).shuffle(files)
    if len(files) >= world:
        return files[rank::world]
    return [files[rank % len(files)]]


class ShardPrefetcher:
    """Iterates over shard files while the next one is read and decompressed in the background."""

    def __init__(self, files: Sequence[str], max_pred_length: Optional[int] = None):
        self.files = list(files)
        self.max_pred_length = max_pred_length
        self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="shard-prefetch")

    def __iter__(self) -> Iterator[PretrainingShard]:
        pending: Optional[Future] = self._pool.submit(load_shard, self.files[0]) if self.files else None
        for k in range(len(self.files)):
            arrays = pending.result()
            pending = self._pool.submit(load_shard, self.files[k + 1]) if k + 1 < len(self.files) else None
            yield PretrainingShard(arrays, self.max_pred_length)

    def close(self) -> None:
        self._pool.shutdown(wait=False, cancel_futures=True)
