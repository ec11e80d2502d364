"""Extractive question answering with the BERT model of this package: one question, one context,
the best answer spans as JSON.

Counterpart of the reference's ``examples/BertPretraining/inference.py`` (features from a
question/context pair ``:57-134``, span selection ``:137-216``): the context is cut to what fits
behind the question, the ``n_best_size`` best start and end positions are paired, pairs that are
out of order, too long or outside the context are dropped, and the rest are ranked by the sum of
their logits.  With ``--version_2_with_negative`` the empty answer competes with its [CLS] score.

    python examples/bert_pretraining/inference.py --vocab_file vocab.txt --bert_model base \
        --init_checkpoint ckpt.pt --question "..." --context "..."
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from conef_b200 import models  # noqa: E402
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402


def build_features(question, context, tokenizer, max_seq_length, max_query_length):
    """``(input_ids, input_mask, segment_ids, tokens, token_to_word, words)``; ``token_to_word[t]`` is
    the index of the whitespace word of the context that token ``t`` came from, or -1."""
    query = tokenizer.tokenize(question)[:max_query_length]
    words = context.split()
    pieces, owner = [], []
    for w_idx, word in enumerate(words):
        for piece in tokenizer.tokenize(word):
            pieces.append(piece)
            owner.append(w_idx)
    room = max_seq_length - len(query) - 3
    pieces, owner = pieces[:room], owner[:room]
    tokens = ["[CLS]"] + query + ["[SEP]"] + pieces + ["[SEP]"]
    segment_ids = [0] * (len(query) + 2) + [1] * (len(pieces) + 1)
    token_to_word = [-1] * (len(query) + 2) + owner + [-1]
    ids = tokenizer.convert_tokens_to_ids(tokens)
    pad = max_seq_length - len(ids)
    return ids + [0] * pad, [1] * len(ids) + [0] * pad, segment_ids + [0] * pad, tokens, token_to_word, words


def best_spans(start_logits, end_logits, token_to_word, words, n_best_size=1, max_answer_length=30,
               with_negative=False, null_score_diff_threshold=0.0):
    """Ranked ``[{"text", "start_logit", "end_logit"}]``; the empty answer is ``text == ""``."""
    n = len(token_to_word)
    top = lambda xs: sorted(range(n), key=lambda i: xs[i], reverse=True)[:n_best_size]
    cands = []
    for s in top(start_logits):
        for e in top(end_logits):
            if token_to_word[s] < 0 or token_to_word[e] < 0 or e < s or e - s + 1 > max_answer_length:
                continue
            text = " ".join(words[token_to_word[s] : token_to_word[e] + 1])
            cands.append({"text": text, "start_logit": float(start_logits[s]), "end_logit": float(end_logits[e])})
    cands.sort(key=lambda c: c["start_logit"] + c["end_logit"], reverse=True)
    if with_negative:
        null = {"text": "", "start_logit": float(start_logits[0]), "end_logit": float(end_logits[0])}
        best = cands[0]["start_logit"] + cands[0]["end_logit"] if cands else float("-inf")
        if null["start_logit"] + null["end_logit"] - best > null_score_diff_threshold:
            cands.insert(0, null)
        else:
            cands.append(null)
    return cands or [{"text": "", "start_logit": 0.0, "end_logit": 0.0}]


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--vocab_file", required=True)
    p.add_argument("--bert_model", default="base", choices=["large", "base", "tiny"])
    p.add_argument("--config_file", default=None)
    p.add_argument("--init_checkpoint", default=None, help="checkpoint with a 'model' state dict")
    p.add_argument("--question", required=True)
    p.add_argument("--context", required=True)
    p.add_argument("--max_seq_length", type=int, default=384)
    p.add_argument("--max_query_length", type=int, default=64)
    p.add_argument("--n_best_size", type=int, default=1)
    p.add_argument("--max_answer_length", type=int, default=30)
    p.add_argument("--version_2_with_negative", action="store_true")
    p.add_argument("--null_score_diff_threshold", type=float, default=0.0)
    p.add_argument("--do_lower_case", action="store_true", default=True)
    p.add_argument("--bf16", action="store_true")
    p.add_argument("--no_cuda", action="store_true")
    p.add_argument("--seed", type=int, default=1)
    args = p.parse_args()

    torch.manual_seed(args.seed)
    device = torch.device("cuda" if torch.cuda.is_available() and not args.no_cuda else "cpu")
    tok = BertTokenizer(args.vocab_file, do_lower_case=args.do_lower_case)
    if args.config_file:
        cfg = models.BertConfig.from_json_file(args.config_file)
    elif args.bert_model == "large":
        cfg = models.BertConfig.large()
    elif args.bert_model == "base":
        cfg = models.BertConfig.base()
    else:
        cfg = models.BertConfig(max(len(tok.vocab), 8), hidden_size=128, num_hidden_layers=2,
                                num_attention_heads=4, intermediate_size=512)
    net = models.BertForQuestionAnswering(cfg)
    if args.init_checkpoint:
        sd = torch.load(args.init_checkpoint, map_location="cpu")
        missing, unexpected = net.load_state_dict(sd.get("model", sd), strict=False)
        print(f"loaded {args.init_checkpoint}: {len(missing)} missing, {len(unexpected)} unexpected keys", file=sys.stderr)
    net = net.to(device).eval()
    ids, mask, seg, tokens, token_to_word, words = build_features(args.question, args.context, tok,
                                                                   args.max_seq_length, args.max_query_length)
    t = lambda x: torch.tensor([x], device=device)
    amp = torch.autocast("cuda", dtype=torch.bfloat16) if (args.bf16 and device.type == "cuda") \
        else torch.autocast("cpu", enabled=False)
    with torch.no_grad(), amp:
        start, end = net(t(ids), t(seg), t(mask))
    n = len(tokens)
    answers = best_spans(start[0, :n].float().tolist(), end[0, :n].float().tolist(), token_to_word, words,
                         args.n_best_size, args.max_answer_length, args.version_2_with_negative,
                         args.null_score_diff_threshold)
    print(json.dumps({"question": args.question, "answers": answers}))


if __name__ == "__main__":
    main()
