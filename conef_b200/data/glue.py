"""GLUE-style sentence(-pair) classification data: TSV readers and BERT input features.

Same surface as the reference's ``examples/BertPretraining/processors/glue.py`` (``InputExample``
``:22-41``, ``InputFeatures`` ``:44-51``, one processor per task ``:82-227``,
``convert_examples_to_features`` ``:230-300``), but table driven: a task is a row of column
indices, not a class body.  None of this touches gradient compression; it exists so that the BERT
model of this package can be fine-tuned or probed from the same kind of files.
"""
from __future__ import annotations

import csv
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence


@dataclass
class InputExample:
    guid: str
    text_a: str
    text_b: Optional[str] = None
    label: Optional[str] = None


@dataclass
class InputFeatures:
    input_ids: List[int]
    input_mask: List[int]
    segment_ids: List[int]
    label_id: Optional[int]


@dataclass(frozen=True)
class TaskSpec:
    """Where a task keeps its fields in ``train.tsv`` / ``dev.tsv`` (dev file name may differ)."""
    labels: Sequence[str]
    text_a: int
    text_b: Optional[int]
    label: int
    header: bool = True
    dev_file: str = "dev.tsv"


TASKS: Dict[str, TaskSpec] = {
    "mrpc": TaskSpec(("0", "1"), text_a=3, text_b=4, label=0),
    "mnli": TaskSpec(("contradiction", "entailment", "neutral"), text_a=8, text_b=9, label=-1,
                     dev_file="dev_matched.tsv"),
    "cola": TaskSpec(("0", "1"), text_a=3, text_b=None, label=1, header=False),
    "sst-2": TaskSpec(("0", "1"), text_a=0, text_b=None, label=1),
}


class DataProcessor:
    """Reads the TSV files of one task."""

    def __init__(self, task: str):
        key = task.lower()
        if key not in TASKS:
            raise KeyError(f"unknown task {task!r}; known: {sorted(TASKS)}")
        self.task, self.spec = key, TASKS[key]

    @staticmethod
    def _read_tsv(path: str, quotechar=None) -> List[List[str]]:
        with open(path, encoding="utf-8") as f:
            return list(csv.reader(f, delimiter="\t", quotechar=quotechar))

    def _examples(self, path: str, set_type: str) -> List[InputExample]:
        rows = self._read_tsv(path)
        if self.spec.header:
            rows = rows[1:]
        out = []
        for i, row in enumerate(rows):
            if not row:
                continue
            text_b = row[self.spec.text_b] if self.spec.text_b is not None else None
            out.append(InputExample(f"{set_type}-{i}", row[self.spec.text_a], text_b, row[self.spec.label]))
        return out

    def get_train_examples(self, data_dir: str) -> List[InputExample]:
        return self._examples(os.path.join(data_dir, "train.tsv"), "train")

    def get_dev_examples(self, data_dir: str) -> List[InputExample]:
        return self._examples(os.path.join(data_dir, self.spec.dev_file), "dev")

    def get_labels(self) -> List[str]:
        return list(self.spec.labels)


PROCESSORS = {name: (lambda name=name: DataProcessor(name)) for name in TASKS}


def truncate_seq_pair(tokens_a: List[str], tokens_b: List[str], max_length: int) -> None:
    """Drop tokens from the end of the longer sequence until the pair fits."""
    while len(tokens_a) + len(tokens_b) > max_length:
        (tokens_a if len(tokens_a) > len(tokens_b) else tokens_b).pop()


def encode_pair(tokenizer, text_a: str, text_b: Optional[str], max_seq_length: int):
    """``[CLS] a [SEP]`` or ``[CLS] a [SEP] b [SEP]`` padded to ``max_seq_length``:
    ``(tokens, input_ids, input_mask, segment_ids)``."""
    a = tokenizer.tokenize(text_a)
    b = tokenizer.tokenize(text_b) if text_b else None
    if b is not None:
        truncate_seq_pair(a, b, max_seq_length - 3)
    else:
        a = a[: max_seq_length - 2]
    tokens = ["[CLS]"] + a + ["[SEP]"]
    segment_ids = [0] * len(tokens)
    if b is not None:
        tokens += b + ["[SEP]"]
        segment_ids += [1] * (len(b) + 1)
    input_ids = tokenizer.convert_tokens_to_ids(tokens)
    pad = max_seq_length - len(input_ids)
    input_mask = [1] * len(input_ids) + [0] * pad
    return tokens, input_ids + [0] * pad, input_mask, segment_ids + [0] * pad


def convert_examples_to_features(examples: Sequence[InputExample], label_list: Optional[Sequence[str]],
                                 max_seq_length: int, tokenizer) -> List[InputFeatures]:
    label_map = {label: i for i, label in enumerate(label_list)} if label_list else {}
    out = []
    for ex in examples:
        _, ids, mask, seg = encode_pair(tokenizer, ex.text_a, ex.text_b, max_seq_length)
        out.append(InputFeatures(ids, mask, seg, label_map.get(ex.label) if ex.label is not None else None))
    return out
