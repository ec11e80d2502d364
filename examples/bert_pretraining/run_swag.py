"""Fine-tune and evaluate BERT on SWAG-style multiple choice (pick the right ending of four).

The reference ships the launch script of this task (``examples/BertPretraining/scripts/run_swag.sh``:
checkpoint, ``train`` / ``eval`` mode, batch size 12, learning rate 5e-6, two epochs) and the model head
(``modeling.py:1093-1160``), but not the entry point the script calls.  This is that entry point for
``conef_b200.models.BertForMultipleChoice``.  The data files are the task's ``train.csv`` / ``val.csv``
(columns ``sent1``, ``sent2``, ``ending0`` ... ``ending3``, ``label``; the context is ``sent1``, every
choice is ``sent2`` followed by one ending).  Training runs under DistributedDataParallel with any
reducer of the registry; evaluation reports accuracy into ``eval_results.json``.

    torchrun --nproc-per-node 8 examples/bert_pretraining/run_swag.py --do_train --do_eval \
        --data_dir swag --vocab_file vocab.txt --bert_model large --init_checkpoint ckpt_1563.pt
"""
import argparse
import csv
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import finetune as ft  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.data.glue import encode_pair  # noqa: E402
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402


def read_swag(path):
    """``[(context, start_of_ending, [endings], label or None)]``; the number of ``ending<k>`` columns is
    the number of choices."""
    rows = []
    with open(path, newline="", encoding="utf-8") as f:
        reader = csv.DictReader(f)
        endings = sorted((c for c in reader.fieldnames if c.startswith("ending")), key=lambda c: int(c[6:]))
        for r in reader:
            label = int(r["label"]) if r.get("label") not in (None, "") else None
            rows.append((r["sent1"], r["sent2"], [r[c] for c in endings], label))
    return rows


def choice_features(rows, tokenizer, max_seq_length):
    """Three ``[N, choices, S]`` lists (ids, segments, mask) and the labels."""
    ids, seg, mask, labels = [], [], [], []
    for context, start, endings, label in rows:
        enc = [encode_pair(tokenizer, context, (start + " " + e).strip(), max_seq_length) for e in endings]
        ids.append([e[1] for e in enc])
        mask.append([e[2] for e in enc])
        seg.append([e[3] for e in enc])
        labels.append(-1 if label is None else label)
    return ids, seg, mask, labels


def parse(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--data_dir", required=True, help="directory with train.csv and val.csv")
    p.add_argument("--output_dir", default="results/swag")
    p.add_argument("--do_train", action="store_true")
    p.add_argument("--do_eval", action="store_true")
    p.add_argument("--eval_batch_size", type=int, default=16)
    ft.add_common_arguments(p, batch=12, lr=5e-6, epochs=2.0, seed=42, max_seq_length=128)
    args = p.parse_args(argv)
    if not (args.do_train or args.do_eval):
        p.error("give --do_train and/or --do_eval")
    ft.check_common_arguments(p, args)
    return args


def main(argv=None):
    args = parse(argv)
    rt = ft.init_runtime(args, args.do_train, port="29509")
    tok = BertTokenizer(args.vocab_file, do_lower_case=args.do_lower_case)
    train_rows = read_swag(os.path.join(args.data_dir, "train.csv")) if args.do_train else []
    eval_rows = read_swag(os.path.join(args.data_dir, "val.csv")) if args.do_eval else []
    choices = len((train_rows or eval_rows)[0][2])
    net = models.BertForMultipleChoice(ft.bert_config(args, len(tok.vocab)), num_choices=choices)
    fresh = ft.load_matching_weights(net, args.init_checkpoint) if args.init_checkpoint else []
    net = net.to(rt.device)
    if rt.rank == 0:
        os.makedirs(args.output_dir, exist_ok=True)
    results = {"world_size": rt.world, "grad_reducer": args.grad_reducer, "num_choices": choices,
               "tensors_not_in_checkpoint": len(fresh)}

    if args.do_train:
        ids, seg, mask, lab = (rt.tensor(x) for x in choice_features(train_rows, tok, args.max_seq_length))
        results.update(ft.train(net, args, rt, len(train_rows),
                                lambda model, i: F.cross_entropy(model(ids[i], seg[i], mask[i]).float(), lab[i])))
        if rt.rank == 0:
            torch.save({"model": net.state_dict()}, os.path.join(args.output_dir, "pytorch_model.pt"))

    if args.do_eval and rt.rank == 0:
        ids, seg, mask, lab = (rt.tensor(x) for x in choice_features(eval_rows, tok, args.max_seq_length))
        net.eval()
        hits, loss_sum = 0, 0.0
        with torch.no_grad():
            for lo in range(0, len(eval_rows), args.eval_batch_size):
                sl = slice(lo, lo + args.eval_batch_size)
                with rt.amp():
                    logits = net(ids[sl], seg[sl], mask[sl]).float()
                loss_sum += float(F.cross_entropy(logits, lab[sl], reduction="sum"))
                hits += int((logits.argmax(-1) == lab[sl]).sum())
        results.update({"eval_examples": len(eval_rows), "eval_loss": loss_sum / max(len(eval_rows), 1),
                        "eval_accuracy": hits / max(len(eval_rows), 1)})
    if rt.rank == 0:
        with open(os.path.join(args.output_dir, "eval_results.json"), "w") as f:
            json.dump(results, f, indent=1)
        print(json.dumps(results))
    ft.finish(rt)
    return results


if __name__ == "__main__":
    main()
