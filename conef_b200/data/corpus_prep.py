"""Offline corpus preparation for BERT pre-training: formatting, sentence segmentation, sharding.

Counterparts in the reference (vendored NVIDIA scripts, ``examples/BertPretraining/data/``):
``WikicorpusTextFormatting.py`` (wikiextractor output -> one article per line),
``BookscorpusTextFormatting.py`` (one book per file -> one book per line), ``TextSharding.py``
(articles -> sentences -> balanced training / test shards, ``Sharding`` :20-316, sentence
segmentation with NLTK :318-327) and the ``text_formatting`` / ``sharding`` actions of
``bertPrep.py:27-363``.  Everything here works from local files; downloading corpora is not part of
it (the machines this library runs on have no network), and sentences are split by a rule-based
segmenter because NLTK's ``punkt`` model is a download as well.

File formats: formatted corpora hold one article per line; shards hold one sentence per line with
a blank line between articles, which is what ``create_pretraining_data.py`` reads.
"""
from __future__ import annotations

import glob
import heapq
import os
import re
from typing import Dict, Iterable, Iterator, List, Sequence, Tuple


# -- formatting -------------------------------------------------------------
def iter_wikiextractor_articles(paths: Iterable[str]) -> Iterator[str]:
    """Articles of wikiextractor output (``<doc id=... title=...>`` ... ``</doc>`` blocks, the first
    line of a block being the title): the body joined into one line."""
    for path in paths:
        body, inside, first = [], False, False
        with open(path, encoding="utf-8", errors="replace", newline="\n") as f:
            for line in f:
                if line.startswith("<doc id="):
                    body, inside, first = [], True, True
                elif line.startswith("</doc>"):
                    if body:
                        yield " ".join(body)
                    inside = False
                elif inside:
                    if first:                    # the title line
                        first = False
                        continue
                    text = line.strip()
                    if text:
                        body.append(text)


def format_wikicorpus(input_dir: str, output_file: str, recursive: bool = True) -> int:
    """``input_dir``: a wikiextractor output tree (files named ``wiki_*``).  Returns the article count."""
    pattern = os.path.join(input_dir, "**", "wiki_*") if recursive else os.path.join(input_dir, "wiki_*")
    paths = sorted(glob.glob(pattern, recursive=recursive))
    n = 0
    with open(output_file, "w", encoding="utf-8", newline="\n") as out:
        for article in iter_wikiextractor_articles(paths):
            out.write(article + "\n")
            n += 1
    return n


def format_bookscorpus(input_dir: str, output_file: str, recursive: bool = True) -> int:
    """Every ``*.txt`` under ``input_dir`` is one book; it becomes one line.  Returns the book count."""
    pattern = os.path.join(input_dir, "**", "*.txt") if recursive else os.path.join(input_dir, "*.txt")
    n = 0
    with open(output_file, "w", encoding="utf-8", newline="\n") as out:
        for path in sorted(glob.glob(pattern, recursive=recursive)):
            with open(path, encoding="utf-8-sig", errors="replace", newline="\n") as f:
                words = [line.strip() for line in f if line.strip()]
            if words:
                out.write(" ".join(words) + "\n")
                n += 1
    return n


# -- sentence segmentation ----------------------------------------------------
_ABBREVIATIONS = {"mr", "mrs", "ms", "dr", "prof", "sr", "jr", "st", "vs", "etc", "e.g", "i.e", "inc", "ltd", "co",
                  "corp", "no", "fig", "al", "approx", "dept", "gen", "gov", "col", "lt", "sgt", "capt", "rev", "u.s",
                  "jan", "feb", "mar", "apr", "jun", "jul", "aug", "sep", "sept", "oct", "nov", "dec"}
_BOUNDARY = re.compile(r"([.!?]+[\"'\)\]]*)\s+(?=[\"'\(\[]*[A-Z0-9])")


class RuleSegmenter:
    """Sentence splitter: a run of ``. ! ?`` (plus closing quotes / brackets) followed by white space
    and an upper-case letter or digit ends a sentence, unless the word before the period is a known
    abbreviation, a single capital (an initial) or a number followed by a lower-case continuation."""

    def segment_string(self, article: str) -> List[str]:
        out, start = [], 0
        for m in _BOUNDARY.finditer(article):
            head = article[start:m.end(1)]
            last = head.rstrip("\"')].!?").rsplit(None, 1)
            word = last[-1].lower() if last else ""
            if m.group(1).startswith(".") and (word in _ABBREVIATIONS or re.fullmatch(r"[a-z]", word)):
                continue
            out.append(head.strip())
            start = m.end()
        tail = article[start:].strip()
        if tail:
            out.append(tail)
        return out


# -- sharding -------------------------------------------------------------------
class Sharding:
    """Articles -> sentences -> ``n_training_shards`` + ``n_test_shards`` text files with about the same
    number of sentences each; ``fraction_test_set`` of all sentences goes to the test shards.

    The assignment is longest-article-first into the shard that is furthest below its target (a
    min-heap of fill levels), which balances tighter than the reference's nominal-size sweep
    (``TextSharding.py:145-283``) and always places every article.  File names follow the reference:
    ``<prefix>_training_<i>.txt`` and ``<prefix>_test_<i>.txt``."""

    def __init__(self, input_files: Sequence[str], output_name_prefix: str, n_training_shards: int,
                 n_test_shards: int, fraction_test_set: float):
        if not input_files:
            raise ValueError("the input file list must contain at least one file")
        if n_training_shards < 1 or n_test_shards < 0:
            raise ValueError("there must be at least one training shard")
        if not 0.0 <= fraction_test_set < 1.0:
            raise ValueError("fraction_test_set must be in [0, 1)")
        self.input_files = list(input_files)
        self.prefix = output_name_prefix
        self.n_train, self.n_test, self.fraction_test = n_training_shards, n_test_shards, fraction_test_set
        self.articles: Dict[int, str] = {}
        self.sentences: Dict[int, List[str]] = {}
        self.output_training_files: Dict[str, List[int]] = {
            f"{self.prefix}_training_{i}.txt": [] for i in range(self.n_train)}
        self.output_test_files: Dict[str, List[int]] = {f"{self.prefix}_test_{i}.txt": [] for i in range(self.n_test)}

    def load_articles(self) -> None:
        n = 0
        for path in self.input_files:
            with open(path, encoding="utf-8", newline="\n") as f:
                for line in f:
                    if line.strip():
                        self.articles[n] = line.rstrip()
                        n += 1

    def segment_articles_into_sentences(self, segmenter=None) -> None:
        if not self.articles:
            self.load_articles()
        if not self.articles:
            raise ValueError("the input files contain no articles")
        segmenter = segmenter or RuleSegmenter()
        for k, article in self.articles.items():
            self.sentences[k] = segmenter.segment_string(article)

    def sentences_per_shard(self, shard: Sequence[int]) -> int:
        return sum(len(self.sentences[a]) for a in shard)

    def distribute_articles_over_shards(self) -> None:
        if not self.sentences:
            self.segment_articles_into_sentences()
        if len(self.articles) < self.n_train + self.n_test:
            raise ValueError("there are fewer articles than shards: add data or ask for fewer shards")
        total = sum(len(s) for s in self.sentences.values())
        test_total = self.fraction_test * total if self.n_test else 0.0
        targets: List[Tuple[str, float]] = [(name, (total - test_total) / self.n_train)
                                            for name in self.output_training_files]
        targets += [(name, test_total / self.n_test) for name in self.output_test_files]
        files = {**self.output_training_files, **self.output_test_files}
        # heap of (fill relative to target, tie-break, name, target)
        heap = [(0.0, i, name, max(t, 1e-9)) for i, (name, t) in enumerate(targets)]
        heapq.heapify(heap)
        order = sorted(self.sentences, key=lambda a: (-len(self.sentences[a]), a))
        # every shard gets one article first (the longest ones), then the emptiest shard gets the next
        for a in order:
            fill, i, name, target = heapq.heappop(heap)
            files[name].append(a)
            heapq.heappush(heap, (fill + max(len(self.sentences[a]), 1) / target, i, name, target))

    def write_shards_to_disk(self) -> List[str]:
        written = []
        for name, shard in {**self.output_training_files, **self.output_test_files}.items():
            os.makedirs(os.path.dirname(os.path.abspath(name)), exist_ok=True)
            with open(name, "w", encoding="utf-8", newline="\n") as f:
                for a in shard:
                    for sentence in self.sentences[a]:
                        f.write(sentence + "\n")
                    f.write("\n")                 # a blank line between articles
            written.append(name)
        return written
