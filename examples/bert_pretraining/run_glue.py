"""Fine-tune and evaluate BERT on a GLUE sentence(-pair) classification task.

The reference ships the launch script for this (``examples/BertPretraining/scripts/run_glue.sh``:
task, data directory, vocabulary, checkpoint, batch size, learning rate, warm-up proportion, epochs,
``train`` / ``eval`` modes) and the task processors (``processors/glue.py``), but not the entry point
the script calls.  This is that entry point for the BERT model of this package: weights start from a
pre-training checkpoint (the encoder's tensors are taken, the classifier starts fresh), training runs
under DistributedDataParallel with any reducer of the registry (``--grad_reducer``, plain all-reduce by
default: fine-tuning runs are short), evaluation reports accuracy, F1 (MRPC) and Matthews correlation
(CoLA) into ``eval_results.json``.

    torchrun --nproc-per-node 8 examples/bert_pretraining/run_glue.py --task_name mrpc --do_train --do_eval \
        --data_dir glue/MRPC --vocab_file vocab.txt --bert_model large --init_checkpoint ckpt_7038.pt \
        --output_dir results/MRPC
"""
import argparse
import json
import math
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import finetune as ft  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.data import glue  # noqa: E402
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402


def parse(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--task_name", required=True, choices=sorted(glue.PROCESSORS))
    p.add_argument("--data_dir", required=True, help="directory with the task's train.tsv and dev file")
    p.add_argument("--output_dir", default="results/glue")
    p.add_argument("--do_train", action="store_true")
    p.add_argument("--do_eval", action="store_true")
    p.add_argument("--eval_batch_size", type=int, default=32)
    ft.add_common_arguments(p, batch=16, lr=2.4e-5, epochs=3.0, seed=2, max_seq_length=128)
    args = p.parse_args(argv)
    if not (args.do_train or args.do_eval):
        p.error("give --do_train and/or --do_eval")
    ft.check_common_arguments(p, args)
    return args


def to_tensors(features, rt):
    return (rt.tensor([f.input_ids for f in features]), rt.tensor([f.segment_ids for f in features]),
            rt.tensor([f.input_mask for f in features]),
            rt.tensor([f.label_id if f.label_id is not None else -1 for f in features]))


def classification_metrics(task, preds, labels):
    """Accuracy for every task; F1 of the positive class for MRPC; Matthews correlation for CoLA."""
    n = max(len(labels), 1)
    out = {"accuracy": sum(int(p == l) for p, l in zip(preds, labels)) / n}
    if task in ("mrpc", "cola"):
        tp = sum(int(p == 1 and l == 1) for p, l in zip(preds, labels))
        fp = sum(int(p == 1 and l == 0) for p, l in zip(preds, labels))
        fn = sum(int(p == 0 and l == 1) for p, l in zip(preds, labels))
        tn = sum(int(p == 0 and l == 0) for p, l in zip(preds, labels))
        if task == "mrpc":
            out["f1"] = 2 * tp / max(2 * tp + fp + fn, 1)
        else:
            den = math.sqrt(float((tp + fp) * (tp + fn) * (tn + fp) * (tn + fn)))
            out["mcc"] = (tp * tn - fp * fn) / den if den > 0 else 0.0
    return out


def evaluate(net, tensors, batch_size, amp):
    net.eval()
    ids, seg, mask, labels = tensors
    preds, loss_sum = [], 0.0
    with torch.no_grad():
        for lo in range(0, ids.shape[0], batch_size):
            sl = slice(lo, lo + batch_size)
            with amp():
                logits = net(ids[sl], seg[sl], mask[sl])
            loss_sum += float(F.cross_entropy(logits.float(), labels[sl], reduction="sum"))
            preds += logits.argmax(-1).tolist()
    return preds, loss_sum / max(ids.shape[0], 1)


def main(argv=None):
    args = parse(argv)
    rt = ft.init_runtime(args, args.do_train, port="29507")
    tok = BertTokenizer(args.vocab_file, do_lower_case=args.do_lower_case)
    proc = glue.PROCESSORS[args.task_name]()
    labels = proc.get_labels()
    net = models.BertForSequenceClassification(ft.bert_config(args, len(tok.vocab)), num_labels=len(labels))
    fresh = ft.load_matching_weights(net, args.init_checkpoint) if args.init_checkpoint else []
    net = net.to(rt.device)
    if rt.rank == 0:
        os.makedirs(args.output_dir, exist_ok=True)
    results = {"task": args.task_name, "world_size": rt.world, "grad_reducer": args.grad_reducer,
               "tensors_not_in_checkpoint": len(fresh)}

    if args.do_train:
        feats = glue.convert_examples_to_features(proc.get_train_examples(args.data_dir), labels,
                                                  args.max_seq_length, tok)
        ids, seg, mask, lab = to_tensors(feats, rt)
        results.update(ft.train(net, args, rt, len(feats),
                                lambda model, i: F.cross_entropy(model(ids[i], seg[i], mask[i]).float(), lab[i])))
        if rt.rank == 0:
            torch.save({"model": net.state_dict(), "task": args.task_name, "labels": list(labels)},
                       os.path.join(args.output_dir, "pytorch_model.pt"))

    if args.do_eval and rt.rank == 0:
        feats = glue.convert_examples_to_features(proc.get_dev_examples(args.data_dir), labels,
                                                  args.max_seq_length, tok)
        tensors = to_tensors(feats, rt)
        preds, loss = evaluate(net, tensors, args.eval_batch_size, rt.amp)
        metrics = classification_metrics(args.task_name, preds, tensors[3].tolist())
        results.update({"eval_examples": len(feats), "eval_loss": loss, **{"eval_" + k: v for k, v in metrics.items()}})
    if rt.rank == 0:
        with open(os.path.join(args.output_dir, "eval_results.json"), "w") as f:
            json.dump(results, f, indent=1)
        print(json.dumps(results))
    ft.finish(rt)
    return results


if __name__ == "__main__":
    main()
