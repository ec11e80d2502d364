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
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import conef_b200 as cb  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.data import glue  # noqa: E402
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402
from conef_b200.optim import BertAdam  # noqa: E402


def parse(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--task_name", required=True, choices=sorted(glue.PROCESSORS))
    p.add_argument("--data_dir", required=True, help="directory with the task's train.tsv and dev file")
    p.add_argument("--vocab_file", required=True)
    p.add_argument("--bert_model", default="large", choices=["large", "base", "tiny"])
    p.add_argument("--config_file", default=None)
    p.add_argument("--init_checkpoint", default=None,
                   help="pre-training or fine-tuned checkpoint ('model' state dict); random weights without")
    p.add_argument("--output_dir", default="results/glue")
    p.add_argument("--do_train", action="store_true")
    p.add_argument("--do_eval", action="store_true")
    p.add_argument("--do_lower_case", action="store_true", default=True)
    p.add_argument("--max_seq_length", type=int, default=128)
    p.add_argument("--train_batch_size", type=int, default=16, help="per process, per optimizer step")
    p.add_argument("--eval_batch_size", type=int, default=32)
    p.add_argument("--gradient_accumulation_steps", type=int, default=1)
    p.add_argument("--learning_rate", type=float, default=2.4e-5)
    p.add_argument("--warmup_proportion", type=float, default=0.1)
    p.add_argument("--num_train_epochs", type=float, default=3.0)
    p.add_argument("--max_steps", type=int, default=-1, help="stop after this many optimizer steps when positive")
    p.add_argument("--bf16", action="store_true")
    p.add_argument("--no_cuda", action="store_true")
    p.add_argument("--seed", type=int, default=2)
    p.add_argument("--grad_reducer", default="allreduce", choices=cb.REDUCERS)
    p.add_argument("--start_compression_percentage", type=float, default=0.1)
    p.add_argument("--compression_ratio", type=float, default=0.1)
    p.add_argument("--sketch_size", type=float, default=0.1)
    p.add_argument("--beta", type=float, default=0.9)
    p.add_argument("--matrix_approximation_rank", type=int, default=8)
    p.add_argument("--min_compression_rate", type=float, default=2)
    p.add_argument("--orthogonalization_epsilon", type=float, default=0)
    p.add_argument("--error_compressor", default=None)
    p.add_argument("--local_rank", type=int, default=int(os.environ.get("LOCAL_RANK", 0)))
    args = p.parse_args(argv)
    if not (args.do_train or args.do_eval):
        p.error("give --do_train and/or --do_eval")
    if args.gradient_accumulation_steps < 1 or args.train_batch_size % args.gradient_accumulation_steps:
        p.error("--train_batch_size must be a positive multiple of --gradient_accumulation_steps")
    return args


def to_tensors(features, device):
    t = lambda rows, dtype=torch.long: torch.tensor(rows, dtype=dtype, device=device)
    return (t([f.input_ids for f in features]), t([f.segment_ids for f in features]),
            t([f.input_mask for f in features]), t([f.label_id if f.label_id is not None else -1 for f in features]))


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


def load_encoder_weights(net, path):
    """Take every tensor of the checkpoint whose name and shape match (a pre-training checkpoint has no
    classifier; a fine-tuned one has all of them); returns the names left at their initial values."""
    blob = torch.load(path, map_location="cpu", weights_only=False)
    sd = blob.get("model", blob)
    own = net.state_dict()
    take = {k: v for k, v in sd.items() if k in own and tuple(v.shape) == tuple(own[k].shape)}
    net.load_state_dict(take, strict=False)
    return sorted(set(own) - set(take))


def build_model(args, num_labels, vocab_size):
    if args.config_file:
        cfg = models.BertConfig.from_json_file(args.config_file)
    elif args.bert_model == "large":
        cfg = models.BertConfig.large()
    elif args.bert_model == "base":
        cfg = models.BertConfig.base()
    else:
        cfg = models.BertConfig(max(vocab_size, 8), hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                intermediate_size=512)
    if cfg.vocab_size % 8 != 0:                 # pre-training pads the vocabulary to a multiple of 8
        cfg.vocab_size += 8 - cfg.vocab_size % 8
    return models.BertForSequenceClassification(cfg, num_labels=num_labels)


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
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    cuda = torch.cuda.is_available() and not args.no_cuda
    device = torch.device("cuda", max(args.local_rank, 0)) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    use_ddp = args.do_train and (world > 1 or args.grad_reducer != "allreduce")
    own_group = False
    if use_ddp and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29507")
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
        own_group = True
    torch.manual_seed(args.seed)
    tok = BertTokenizer(args.vocab_file, do_lower_case=args.do_lower_case)
    proc = glue.PROCESSORS[args.task_name]()
    labels = proc.get_labels()
    net = build_model(args, len(labels), len(tok.vocab))
    fresh = []
    if args.init_checkpoint:
        fresh = load_encoder_weights(net, args.init_checkpoint)
    net = net.to(device)
    amp = (lambda: torch.autocast("cuda", dtype=torch.bfloat16)) if (args.bf16 and cuda) \
        else (lambda: torch.autocast("cpu", enabled=False))
    if rank == 0:
        os.makedirs(args.output_dir, exist_ok=True)
    results = {"task": args.task_name, "world_size": world, "grad_reducer": args.grad_reducer,
               "tensors_not_in_checkpoint": len(fresh)}

    if args.do_train:
        feats = glue.convert_examples_to_features(proc.get_train_examples(args.data_dir), labels,
                                                  args.max_seq_length, tok)
        ids, seg, mask, lab = to_tensors(feats, device)
        per_rank = len(feats) // world                      # every rank takes the same number of examples
        steps_per_epoch = max(per_rank // args.train_batch_size, 1)
        total = int(steps_per_epoch * args.num_train_epochs)
        if args.max_steps > 0:
            total = min(total, args.max_steps)
        total = max(total, 1)
        args.start_compression_iter = max(2, int(total * args.start_compression_percentage))
        decay = [p for n, p in net.named_parameters() if p.dim() > 1]
        no_decay = [p for n, p in net.named_parameters() if p.dim() <= 1]
        opt = BertAdam([{"params": decay, "weight_decay": 0.01}, {"params": no_decay, "weight_decay": 0.0}],
                       lr=args.learning_rate, warmup=args.warmup_proportion, t_total=total)
        model, state = net, None
        if use_ddp:
            model = DDP(net, device_ids=[device.index] if cuda else None, gradient_as_bucket_view=True)
            state = cb.get_comm_hooks(args, model, args.local_rank)
        micro = args.train_batch_size // args.gradient_accumulation_steps
        step, t0, losses = 0, time.time(), []
        while step < total:
            epoch = step // steps_per_epoch
            g = torch.Generator().manual_seed(args.seed + epoch)          # same permutation on every rank
            order = torch.randperm(len(feats), generator=g)[rank::world][:per_rank].to(device)
            for b in range(steps_per_epoch):
                if step >= total:
                    break
                net.train()
                idx = order[b * args.train_batch_size:(b + 1) * args.train_batch_size]
                opt.zero_grad(set_to_none=True)
                loss_value = 0.0
                for a in range(args.gradient_accumulation_steps):
                    part = idx[a * micro:(a + 1) * micro]
                    if part.numel() == 0:
                        continue
                    last = a == args.gradient_accumulation_steps - 1
                    sync = model.no_sync if (use_ddp and not last) else _null
                    with sync(), amp():
                        logits = model(ids[part], seg[part], mask[part])
                        loss = F.cross_entropy(logits.float(), lab[part]) / args.gradient_accumulation_steps
                    loss.backward()
                    loss_value += float(loss.detach())
                opt.step()
                losses.append(loss_value)
                step += 1
        if state is not None and hasattr(state, "check_status"):
            state.check_status()
        results.update({"train_steps": step, "train_loss_first": losses[0],
                        "train_loss_last": sum(losses[-10:]) / len(losses[-10:]),      # mean of the last ten steps
                        "train_seq_per_s": step * args.train_batch_size * world / max(time.time() - t0, 1e-9)})
        if rank == 0:
            torch.save({"model": net.state_dict(), "task": args.task_name, "labels": list(labels)},
                       os.path.join(args.output_dir, "pytorch_model.pt"))

    if args.do_eval and rank == 0:
        feats = glue.convert_examples_to_features(proc.get_dev_examples(args.data_dir), labels,
                                                  args.max_seq_length, tok)
        tensors = to_tensors(feats, device)
        preds, loss = evaluate(net, tensors, args.eval_batch_size, amp)
        results.update({"eval_examples": len(feats), "eval_loss": loss,
                        **{"eval_" + k: v for k, v in classification_metrics(args.task_name, preds, tensors[3].tolist()).items()}})
    if rank == 0:
        with open(os.path.join(args.output_dir, "eval_results.json"), "w") as f:
            json.dump(results, f, indent=1)
        print(json.dumps(results))
    if dist.is_initialized():
        dist.barrier()
        if own_group:
            dist.destroy_process_group()
    return results


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


if __name__ == "__main__":
    main()
