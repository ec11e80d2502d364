"""SQuAD-style extractive question answering data: examples, windowed BERT features, answers, scores.

The reference ships the launch script and presets for this task
(``examples/BertPretraining/scripts/run_squad.sh``, ``scripts/configs/squad_config.sh``:
``doc_stride 128``, ``max_seq_length 384``, ``max_query_length 64``, ``n_best_size 20``,
``max_answer_length 30``, v1.1 and v2.0) and a single-pair inference script
(``inference.py:57-216``), but not the training entry point or its data code.  This module is
that data code for ``examples/bert_pretraining/run_squad.py``:

* a context is split on whitespace; the gold answer's character span becomes a word span;
* words become word pieces; a context longer than the room behind the question is cut into
  windows that advance by ``doc_stride`` pieces, and each piece knows the window in which it has
  the most context on both sides (only there may it start or end a predicted answer);
* a window that does not hold the whole gold answer is trained towards position 0 ([CLS]);
* predicted answers are the original words between the best (start, end) pair over all windows
  of a question; with ``with_negative`` the empty answer competes with its best [CLS] score.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


@dataclass
class SquadExample:
    qas_id: str
    question: str
    words: List[str]
    answer_text: Optional[str] = None
    start_word: int = -1
    end_word: int = -1
    is_impossible: bool = False
    gold_texts: List[str] = field(default_factory=list)


@dataclass
class SquadFeatures:
    example_index: int
    window: int
    tokens: List[str]
    token_to_word: List[int]          # -1 outside the context
    max_context: List[bool]           # this window is the best one for the piece at this position
    input_ids: List[int]
    input_mask: List[int]
    segment_ids: List[int]
    start_position: int = 0
    end_position: int = 0


def split_context(context: str) -> Tuple[List[str], List[int]]:
    """Whitespace words of ``context`` and, per character, the index of the word it belongs to
    (a whitespace character belongs to the word before it)."""
    words, char_to_word = [], []
    in_word = False
    for ch in context:
        if ch.isspace() or ch == " ":
            in_word = False
        elif in_word:
            words[-1] += ch
        else:
            words.append(ch)
            in_word = True
        char_to_word.append(len(words) - 1)
    return words, char_to_word


def read_squad_examples(path: str, is_training: bool, with_negative: bool = False) -> List[SquadExample]:
    """Examples of a SQuAD v1.1 / v2.0 JSON file.  For training, an answer whose text cannot be found
    at its character offset (a mis-annotated span) is skipped, as the public BERT recipe does."""
    out = []
    for article in json.load(open(path, encoding="utf-8"))["data"]:
        for para in article["paragraphs"]:
            words, char_to_word = split_context(para["context"])
            for qa in para["qas"]:
                ex = SquadExample(qa["id"], qa["question"], words)
                ex.is_impossible = bool(with_negative and qa.get("is_impossible", False))
                answers = qa.get("answers", [])
                ex.gold_texts = [a["text"] for a in answers]
                if is_training:
                    if not ex.is_impossible:
                        if not answers:
                            continue
                        a = answers[0]
                        start, length = a["answer_start"], len(a["text"])
                        if length == 0 or start + length > len(char_to_word):
                            continue
                        ex.answer_text = a["text"]
                        ex.start_word, ex.end_word = char_to_word[start], char_to_word[start + length - 1]
                        found = " ".join(words[ex.start_word:ex.end_word + 1])
                        if " ".join(a["text"].split()) not in found:
                            continue
                    else:
                        ex.answer_text = ""
                out.append(ex)
    return out


def _narrow_to_answer(pieces: Sequence[str], lo: int, hi: int, tokenizer, answer: str) -> Tuple[int, int]:
    """The tightest piece span inside ``[lo, hi]`` that spells the tokenised answer (a word such as
    ``(1895-1943).`` holds the answer ``1895`` as one of several pieces)."""
    target = " ".join(tokenizer.tokenize(answer))
    for s in range(lo, hi + 1):
        for e in range(hi, s - 1, -1):
            if " ".join(pieces[s:e + 1]) == target:
                return s, e
    return lo, hi


def convert_examples_to_features(examples: Sequence[SquadExample], tokenizer, max_seq_length: int = 384,
                                 doc_stride: int = 128, max_query_length: int = 64,
                                 is_training: bool = False) -> List[SquadFeatures]:
    feats: List[SquadFeatures] = []
    for ex_idx, ex in enumerate(examples):
        query = tokenizer.tokenize(ex.question)[:max_query_length]
        pieces, owner, first_piece = [], [], []
        for w_idx, word in enumerate(ex.words):
            first_piece.append(len(pieces))
            for piece in tokenizer.tokenize(word):
                pieces.append(piece)
                owner.append(w_idx)
        ans_lo = ans_hi = -1
        if is_training and not ex.is_impossible:
            ans_lo = first_piece[ex.start_word]
            ans_hi = (first_piece[ex.end_word + 1] if ex.end_word + 1 < len(ex.words) else len(pieces)) - 1
            ans_lo, ans_hi = _narrow_to_answer(pieces, ans_lo, ans_hi, tokenizer, ex.answer_text)
        room = max_seq_length - len(query) - 3
        if room <= 0:
            raise ValueError("max_seq_length leaves no room for the context behind the question")
        starts, pos = [], 0
        while True:
            starts.append(pos)
            if pos + room >= len(pieces):
                break
            pos += min(room, doc_stride)
        spans = [(s, min(room, len(pieces) - s)) for s in starts]
        # the window in which a piece has the most context: the larger min(left, right), longer windows first
        best_window: Dict[int, int] = {}
        for p in range(len(pieces)):
            best, best_score = -1, -1.0
            for w, (s, n) in enumerate(spans):
                if s <= p < s + n:
                    score = min(p - s, s + n - 1 - p) + 0.01 * n
                    if score > best_score:
                        best, best_score = w, score
            best_window[p] = best
        offset = len(query) + 2
        for w, (s, n) in enumerate(spans):
            tokens = ["[CLS]"] + query + ["[SEP]"] + pieces[s:s + n] + ["[SEP]"]
            segment_ids = [0] * offset + [1] * (n + 1)
            token_to_word = [-1] * offset + owner[s:s + n] + [-1]
            max_context = [False] * offset + [best_window[p] == w for p in range(s, s + n)] + [False]
            ids = tokenizer.convert_tokens_to_ids(tokens)
            pad = max_seq_length - len(ids)
            f = SquadFeatures(ex_idx, w, tokens, token_to_word, max_context, ids + [0] * pad,
                              [1] * len(ids) + [0] * pad, segment_ids + [0] * pad)
            if is_training and not ex.is_impossible and s <= ans_lo and ans_hi < s + n:
                f.start_position, f.end_position = ans_lo - s + offset, ans_hi - s + offset
            feats.append(f)
    return feats


def best_answers(examples: Sequence[SquadExample], features: Sequence[SquadFeatures],
                 start_logits: Sequence[Sequence[float]], end_logits: Sequence[Sequence[float]],
                 n_best_size: int = 20, max_answer_length: int = 30, with_negative: bool = False,
                 null_score_diff_threshold: float = 0.0) -> Tuple[Dict[str, str], Dict[str, List[dict]]]:
    """``({id: answer text}, {id: ranked candidates})`` from the logits of every window
    (``start_logits[i]`` belongs to ``features[i]``)."""
    by_example: Dict[int, List[int]] = {}
    for i, f in enumerate(features):
        by_example.setdefault(f.example_index, []).append(i)
    answers, ranked = {}, {}
    for ex_idx, ex in enumerate(examples):
        cands, null_score = [], float("inf")
        for i in by_example.get(ex_idx, []):
            f, sl, el = features[i], start_logits[i], end_logits[i]
            n = len(f.tokens)
            null_score = min(null_score, float(sl[0]) + float(el[0]))
            top = lambda xs: sorted(range(n), key=lambda j: xs[j], reverse=True)[:n_best_size]
            for s in top(sl):
                for e in top(el):
                    if f.token_to_word[s] < 0 or f.token_to_word[e] < 0 or not f.max_context[s]:
                        continue
                    if e < s or e - s + 1 > max_answer_length:
                        continue
                    cands.append({"text": " ".join(ex.words[f.token_to_word[s]:f.token_to_word[e] + 1]),
                                  "score": float(sl[s]) + float(el[e])})
        cands.sort(key=lambda c: c["score"], reverse=True)
        seen, unique = set(), []
        for c in cands:
            if c["text"] not in seen:
                seen.add(c["text"])
                unique.append(c)
        unique = unique[:n_best_size]
        best = unique[0]["text"] if unique else ""
        if with_negative:
            unique.append({"text": "", "score": null_score})
            if not unique[:-1] or null_score - unique[0]["score"] > null_score_diff_threshold:
                best = ""
        answers[ex.qas_id], ranked[ex.qas_id] = best, unique or [{"text": "", "score": 0.0}]
    return answers, ranked


def _normalise_answer(text: str) -> List[str]:
    text = "".join(ch for ch in text.lower() if ch.isalnum() or ch.isspace())
    return [w for w in text.split() if w not in ("a", "an", "the")]


def squad_scores(predictions: Dict[str, str], path: str) -> Dict[str, float]:
    """Exact match and F1 (percent) of ``{id: text}`` against the gold answers of a SQuAD file, with the
    benchmark's answer normalisation (case, punctuation and articles ignored; best score over the golds;
    a question without gold answers expects the empty answer)."""
    em = f1 = n = 0
    for article in json.load(open(path, encoding="utf-8"))["data"]:
        for para in article["paragraphs"]:
            for qa in para["qas"]:
                golds = [a["text"] for a in qa.get("answers", [])] or [""]
                pred = _normalise_answer(predictions.get(qa["id"], ""))
                best_em = best_f1 = 0.0
                for g in golds:
                    gold = _normalise_answer(g)
                    best_em = max(best_em, float(pred == gold))
                    common = sum(min(pred.count(w), gold.count(w)) for w in set(pred))
                    if not pred or not gold:
                        score = float(pred == gold)
                    elif common == 0:
                        score = 0.0
                    else:
                        prec, rec = common / len(pred), common / len(gold)
                        score = 2 * prec * rec / (prec + rec)
                    best_f1 = max(best_f1, score)
                em, f1, n = em + best_em, f1 + best_f1, n + 1
    return {"exact_match": 100.0 * em / max(n, 1), "f1": 100.0 * f1 / max(n, 1), "questions": n}
