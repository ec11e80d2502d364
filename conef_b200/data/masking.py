"""Masked-LM corruption: 15 % of the positions are predicted; of those 80 % become [MASK],
10 % a random token and 10 % stay unchanged (reference recipe:
``examples/BertPretraining/create_pretraining_data.py:314-364``)."""
from __future__ import annotations

import torch

CLS, SEP, MASK = 101, 102, 103


def mask_tokens(ids: torch.Tensor, vocab: int, prob: float = 0.15, max_predictions: int = 20,
                generator: torch.Generator = None):
    """Returns ``(masked_ids, labels)`` with ``labels == -1`` at positions that are not predicted."""
    ids = ids.clone()
    labels = torch.full_like(ids, -1)
    candidates = ((ids != CLS) & (ids != SEP)).nonzero().flatten()
    n_pred = min(max_predictions, max(1, int(round(len(candidates) * prob))))
    chosen = candidates[torch.randperm(len(candidates), generator=generator)[:n_pred]]
    labels[chosen] = ids[chosen]
    roll = torch.rand(len(chosen), generator=generator)
    ids[chosen[roll < 0.8]] = MASK
    rnd = chosen[(roll >= 0.8) & (roll < 0.9)]
    ids[rnd] = torch.randint(1000, vocab, (len(rnd),), generator=generator)
    return ids, labels
