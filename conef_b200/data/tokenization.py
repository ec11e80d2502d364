"""WordPiece tokenisation for BERT: whitespace / punctuation splitting, optional lower-casing
with accent stripping, then greedy longest-match-first sub-word splitting against a vocabulary
file (one token per line).  Stands in for the reference's vendored
``examples/BertPretraining/tokenization.py`` (392 lines)."""
from __future__ import annotations

import collections
import unicodedata
from typing import Dict, List


def load_vocab(path: str) -> Dict[str, int]:
    vocab = collections.OrderedDict()
    with open(path, "r", encoding="utf-8") as fh:
        for i, line in enumerate(fh):
            vocab[line.rstrip("\n")] = i
    return vocab


def _is_punct(ch: str) -> bool:
    cp = ord(ch)
    if 33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126:
        return True
    return unicodedata.category(ch).startswith("P")


def _is_cjk(cp: int) -> bool:
    return (0x4E00 <= cp <= 0x9FFF or 0x3400 <= cp <= 0x4DBF or 0x20000 <= cp <= 0x2A6DF or 0xF900 <= cp <= 0xFAFF)


class BasicTokenizer:
    def __init__(self, do_lower_case=True, never_split=("[UNK]", "[SEP]", "[PAD]", "[CLS]", "[MASK]")):
        self.do_lower_case, self.never_split = do_lower_case, set(never_split)

    def tokenize(self, text: str) -> List[str]:
        cleaned = []
        for ch in text:
            cp = ord(ch)
            if cp == 0 or cp == 0xFFFD or (unicodedata.category(ch).startswith("C") and ch not in "\t\n\r"):
                continue
            if _is_cjk(cp):
                cleaned.append(f" {ch} ")
            else:
                cleaned.append(" " if ch.isspace() else ch)
        out = []
        for tok in "".join(cleaned).split():
            if tok in self.never_split:
                out.append(tok)
                continue
            if self.do_lower_case:
                tok = "".join(c for c in unicodedata.normalize("NFD", tok.lower()) if unicodedata.category(c) != "Mn")
            cur = ""
            for ch in tok:
                if _is_punct(ch):
                    if cur:
                        out.append(cur)
                    out.append(ch)
                    cur = ""
                else:
                    cur += ch
            if cur:
                out.append(cur)
        return out


class WordpieceTokenizer:
    def __init__(self, vocab, unk_token="[UNK]", max_input_chars_per_word=100):
        self.vocab, self.unk, self.max_chars = vocab, unk_token, max_input_chars_per_word

    def tokenize(self, text: str) -> List[str]:
        out = []
        for tok in text.split():
            if len(tok) > self.max_chars:
                out.append(self.unk)
                continue
            pieces, start, bad = [], 0, False
            while start < len(tok):
                end, cur = len(tok), None
                while start < end:
                    sub = ("##" if start > 0 else "") + tok[start:end]
                    if sub in self.vocab:
                        cur = sub
                        break
                    end -= 1
                if cur is None:
                    bad = True
                    break
                pieces.append(cur)
                start = end
            out.extend([self.unk] if bad else pieces)
        return out


class BertTokenizer:
    def __init__(self, vocab_file: str, do_lower_case=True, max_len=None):
        self.vocab = load_vocab(vocab_file)
        self.ids_to_tokens = {i: t for t, i in self.vocab.items()}
        self.basic = BasicTokenizer(do_lower_case)
        self.wordpiece = WordpieceTokenizer(self.vocab)
        self.max_len = max_len or int(1e12)

    def tokenize(self, text: str) -> List[str]:
        return [p for tok in self.basic.tokenize(text) for p in self.wordpiece.tokenize(tok)]

    def convert_tokens_to_ids(self, tokens: List[str]) -> List[int]:
        ids = [self.vocab.get(t, self.vocab.get("[UNK]", 0)) for t in tokens]
        if len(ids) > self.max_len:
            raise ValueError(f"sequence of {len(ids)} tokens exceeds the model maximum of {self.max_len}")
        return ids

    def convert_ids_to_tokens(self, ids: List[int]) -> List[str]:
        return [self.ids_to_tokens[i] for i in ids]
