"""Fine-tune BERT for extractive question answering on a SQuAD-format file, predict and score.

The reference ships the launch script and presets of this task
(``examples/BertPretraining/scripts/run_squad.sh``, ``scripts/configs/squad_config.sh``) and uses
its result downstream (``triton/deployer.py`` exports the fine-tuned model), but not the entry point
the script calls.  This is that entry point for the BERT model of this package.  Training runs under
DistributedDataParallel with any reducer of the registry (``--grad_reducer``); the loss is the mean
of the cross entropies of the start and the end position; prediction pairs the best start and end
positions over all windows of a question (``conef_b200/data/squad.py``) and writes
``predictions.json`` (+ ``nbest_predictions.json``); ``--do_eval`` scores it against the file's gold
answers (exact match, F1).  The saved ``pytorch_model.pt`` is what ``inference.py`` and
``deploy/export.py`` load with ``--init_checkpoint``.

    torchrun --nproc-per-node 8 examples/bert_pretraining/run_squad.py --do_train --do_predict --do_eval \
        --train_file train-v1.1.json --predict_file dev-v1.1.json --vocab_file vocab.txt \
        --bert_model large --init_checkpoint ckpt_1563.pt --output_dir results/squad
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import finetune as ft  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.data import squad  # noqa: E402
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402


def parse(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--train_file", default=None)
    p.add_argument("--predict_file", default=None)
    p.add_argument("--output_dir", default="results/squad")
    p.add_argument("--do_train", action="store_true")
    p.add_argument("--do_predict", action="store_true")
    p.add_argument("--do_eval", action="store_true", help="score the predictions against --predict_file")
    p.add_argument("--doc_stride", type=int, default=128)
    p.add_argument("--max_query_length", type=int, default=64)
    p.add_argument("--n_best_size", type=int, default=20)
    p.add_argument("--max_answer_length", type=int, default=30)
    p.add_argument("--version_2_with_negative", action="store_true")
    p.add_argument("--null_score_diff_threshold", type=float, default=0.0)
    p.add_argument("--predict_batch_size", type=int, default=8)
    ft.add_common_arguments(p, batch=4, lr=3e-5, epochs=2.0, seed=1, max_seq_length=384)
    args = p.parse_args(argv)
    if not (args.do_train or args.do_predict):
        p.error("give --do_train and/or --do_predict")
    if args.do_train and not args.train_file:
        p.error("--do_train needs --train_file")
    if (args.do_predict or args.do_eval) and not args.predict_file:
        p.error("--do_predict needs --predict_file")
    if args.do_eval and not args.do_predict:
        p.error("--do_eval scores the predictions of --do_predict")
    ft.check_common_arguments(p, args)
    return args


def span_loss(start_logits, end_logits, start_positions, end_positions):
    """Mean of the two cross entropies; positions beyond the sequence are clamped into it."""
    n = start_logits.shape[1]
    return 0.5 * (F.cross_entropy(start_logits.float(), start_positions.clamp(0, n - 1))
                  + F.cross_entropy(end_logits.float(), end_positions.clamp(0, n - 1)))


def main(argv=None):
    args = parse(argv)
    rt = ft.init_runtime(args, args.do_train, port="29508")
    tok = BertTokenizer(args.vocab_file, do_lower_case=args.do_lower_case)
    net = models.BertForQuestionAnswering(ft.bert_config(args, len(tok.vocab)))
    fresh = ft.load_matching_weights(net, args.init_checkpoint) if args.init_checkpoint else []
    for p in net.bert.pooler.parameters():      # the span head reads the token outputs only: the pooler gets no
        p.requires_grad_(False)                 # gradient, which DistributedDataParallel would report as an error
    net = net.to(rt.device)
    if rt.rank == 0:
        os.makedirs(args.output_dir, exist_ok=True)
    results = {"world_size": rt.world, "grad_reducer": args.grad_reducer, "tensors_not_in_checkpoint": len(fresh)}
    inputs = lambda feats: tuple(rt.tensor([getattr(f, k) for f in feats]) for k in ("input_ids", "segment_ids", "input_mask"))

    if args.do_train:
        examples = squad.read_squad_examples(args.train_file, True, args.version_2_with_negative)
        feats = squad.convert_examples_to_features(examples, tok, args.max_seq_length, args.doc_stride,
                                                   args.max_query_length, is_training=True)
        ids, seg, mask = inputs(feats)
        sp, ep = rt.tensor([f.start_position for f in feats]), rt.tensor([f.end_position for f in feats])

        def loss_of(model, i):
            start, end = model(ids[i], seg[i], mask[i])
            return span_loss(start, end, sp[i], ep[i])
        results.update({"train_examples": len(examples), "train_windows": len(feats)})
        results.update(ft.train(net, args, rt, len(feats), loss_of))
        if rt.rank == 0:
            torch.save({"model": net.state_dict()}, os.path.join(args.output_dir, "pytorch_model.pt"))

    sharded = args.do_predict and dist.is_initialized() and rt.world > 1      # every rank scores its share of the windows
    if args.do_predict and (rt.rank == 0 or sharded):
        examples = squad.read_squad_examples(args.predict_file, False, args.version_2_with_negative)
        feats = squad.convert_examples_to_features(examples, tok, args.max_seq_length, args.doc_stride,
                                                   args.max_query_length, is_training=False)
        mine = list(range(rt.rank, len(feats), rt.world)) if sharded else list(range(len(feats)))
        ids, seg, mask = inputs([feats[i] for i in mine])
        net.eval()
        starts, ends, t0 = [], [], time.time()
        with torch.no_grad():
            for lo in range(0, len(mine), args.predict_batch_size):
                sl = slice(lo, lo + args.predict_batch_size)
                with rt.amp():
                    s, e = net(ids[sl], seg[sl], mask[sl])
                starts += s.float().tolist()
                ends += e.float().tolist()
        if sharded:
            parts = [None] * rt.world if rt.rank == 0 else None
            dist.gather_object((mine, starts, ends), parts, dst=0)
            if rt.rank == 0:
                starts, ends = [None] * len(feats), [None] * len(feats)
                for idx, ss, ee in parts:
                    for i, a, b in zip(idx, ss, ee):
                        starts[i], ends[i] = a, b
    if args.do_predict and rt.rank == 0:
        answers, ranked = squad.best_answers(examples, feats, starts, ends, args.n_best_size, args.max_answer_length,
                                             args.version_2_with_negative, args.null_score_diff_threshold)
        with open(os.path.join(args.output_dir, "predictions.json"), "w") as f:
            json.dump(answers, f, indent=1)
        with open(os.path.join(args.output_dir, "nbest_predictions.json"), "w") as f:
            json.dump(ranked, f, indent=1)
        results.update({"predict_questions": len(examples), "predict_windows": len(feats), "predict_ranks": rt.world if sharded else 1,
                        "predict_seq_per_s": len(feats) / max(time.time() - t0, 1e-9)})
        if args.do_eval:
            results.update(squad.squad_scores(answers, args.predict_file))
    if rt.rank == 0:
        with open(os.path.join(args.output_dir, "results.json"), "w") as f:
            json.dump(results, f, indent=1)
        print(json.dumps(results))
    ft.finish(rt)
    return results


if __name__ == "__main__":
    main()
