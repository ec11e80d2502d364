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
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import conef_b200 as cb  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.data import squad  # noqa: E402
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402
from conef_b200.optim import BertAdam  # noqa: E402


def parse(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--train_file", default=None)
    p.add_argument("--predict_file", default=None)
    p.add_argument("--vocab_file", required=True)
    p.add_argument("--bert_model", default="large", choices=["large", "base", "tiny"])
    p.add_argument("--config_file", default=None)
    p.add_argument("--init_checkpoint", default=None)
    p.add_argument("--output_dir", default="results/squad")
    p.add_argument("--do_train", action="store_true")
    p.add_argument("--do_predict", action="store_true")
    p.add_argument("--do_eval", action="store_true", help="score the predictions against --predict_file")
    p.add_argument("--do_lower_case", action="store_true", default=True)
    p.add_argument("--max_seq_length", type=int, default=384)
    p.add_argument("--doc_stride", type=int, default=128)
    p.add_argument("--max_query_length", type=int, default=64)
    p.add_argument("--n_best_size", type=int, default=20)
    p.add_argument("--max_answer_length", type=int, default=30)
    p.add_argument("--version_2_with_negative", action="store_true")
    p.add_argument("--null_score_diff_threshold", type=float, default=0.0)
    p.add_argument("--train_batch_size", type=int, default=4, help="windows per process and optimizer step")
    p.add_argument("--predict_batch_size", type=int, default=8)
    p.add_argument("--gradient_accumulation_steps", type=int, default=1)
    p.add_argument("--learning_rate", type=float, default=3e-5)
    p.add_argument("--warmup_proportion", type=float, default=0.1)
    p.add_argument("--num_train_epochs", type=float, default=2.0)
    p.add_argument("--max_steps", type=int, default=-1)
    p.add_argument("--bf16", action="store_true")
    p.add_argument("--no_cuda", action="store_true")
    p.add_argument("--seed", type=int, default=1)
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
    if not (args.do_train or args.do_predict):
        p.error("give --do_train and/or --do_predict")
    if args.do_train and not args.train_file:
        p.error("--do_train needs --train_file")
    if (args.do_predict or args.do_eval) and not args.predict_file:
        p.error("--do_predict needs --predict_file")
    if args.do_eval and not args.do_predict:
        p.error("--do_eval scores the predictions of --do_predict")
    if args.gradient_accumulation_steps < 1 or args.train_batch_size % args.gradient_accumulation_steps:
        p.error("--train_batch_size must be a positive multiple of --gradient_accumulation_steps")
    return args


def build_model(args, vocab_size):
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
    return models.BertForQuestionAnswering(cfg)


def load_matching_weights(net, path):
    """Take every tensor of the checkpoint whose name and shape match; returns the names left fresh."""
    blob = torch.load(path, map_location="cpu", weights_only=False)
    sd = blob.get("model", blob)
    own = net.state_dict()
    take = {k: v for k, v in sd.items() if k in own and tuple(v.shape) == tuple(own[k].shape)}
    net.load_state_dict(take, strict=False)
    return sorted(set(own) - set(take))


def span_loss(start_logits, end_logits, start_positions, end_positions):
    """Mean of the two cross entropies; positions beyond the sequence are clamped into it."""
    n = start_logits.shape[1]
    return 0.5 * (F.cross_entropy(start_logits.float(), start_positions.clamp(0, n - 1))
                  + F.cross_entropy(end_logits.float(), end_positions.clamp(0, n - 1)))


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


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
        os.environ.setdefault("MASTER_PORT", "29508")
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
        own_group = True
    torch.manual_seed(args.seed)
    tok = BertTokenizer(args.vocab_file, do_lower_case=args.do_lower_case)
    net = build_model(args, len(tok.vocab))
    fresh = load_matching_weights(net, args.init_checkpoint) if args.init_checkpoint else []
    net = net.to(device)
    amp = (lambda: torch.autocast("cuda", dtype=torch.bfloat16)) if (args.bf16 and cuda) \
        else (lambda: torch.autocast("cpu", enabled=False))
    if rank == 0:
        os.makedirs(args.output_dir, exist_ok=True)
    results = {"world_size": world, "grad_reducer": args.grad_reducer, "tensors_not_in_checkpoint": len(fresh)}
    tensor = lambda rows: torch.tensor(rows, dtype=torch.long, device=device)

    if args.do_train:
        examples = squad.read_squad_examples(args.train_file, True, args.version_2_with_negative)
        feats = squad.convert_examples_to_features(examples, tok, args.max_seq_length, args.doc_stride,
                                                   args.max_query_length, is_training=True)
        ids, seg, mask = (tensor([getattr(f, k) for f in feats]) for k in ("input_ids", "segment_ids", "input_mask"))
        sp, ep = tensor([f.start_position for f in feats]), tensor([f.end_position for f in feats])
        per_rank = len(feats) // world
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
                        start, end = model(ids[part], seg[part], mask[part])
                        loss = span_loss(start, end, sp[part], ep[part]) / args.gradient_accumulation_steps
                    loss.backward()
                    loss_value += float(loss.detach())
                opt.step()
                losses.append(loss_value)
                step += 1
        if state is not None and hasattr(state, "check_status"):
            state.check_status()
        results.update({"train_examples": len(examples), "train_windows": len(feats), "train_steps": step,
                        "train_loss_first": losses[0], "train_loss_last": sum(losses[-10:]) / len(losses[-10:]),
                        "train_seq_per_s": step * args.train_batch_size * world / max(time.time() - t0, 1e-9)})
        if rank == 0:
            torch.save({"model": net.state_dict()}, os.path.join(args.output_dir, "pytorch_model.pt"))

    if args.do_predict and rank == 0:
        examples = squad.read_squad_examples(args.predict_file, False, args.version_2_with_negative)
        feats = squad.convert_examples_to_features(examples, tok, args.max_seq_length, args.doc_stride,
                                                   args.max_query_length, is_training=False)
        ids, seg, mask = (tensor([getattr(f, k) for f in feats]) for k in ("input_ids", "segment_ids", "input_mask"))
        net.eval()
        starts, ends, t0 = [], [], time.time()
        with torch.no_grad():
            for lo in range(0, len(feats), args.predict_batch_size):
                sl = slice(lo, lo + args.predict_batch_size)
                with amp():
                    s, e = net(ids[sl], seg[sl], mask[sl])
                starts += s.float().tolist()
                ends += e.float().tolist()
        answers, ranked = squad.best_answers(examples, feats, starts, ends, args.n_best_size, args.max_answer_length,
                                             args.version_2_with_negative, args.null_score_diff_threshold)
        with open(os.path.join(args.output_dir, "predictions.json"), "w") as f:
            json.dump(answers, f, indent=1)
        with open(os.path.join(args.output_dir, "nbest_predictions.json"), "w") as f:
            json.dump(ranked, f, indent=1)
        results.update({"predict_questions": len(examples), "predict_windows": len(feats),
                        "predict_seq_per_s": len(feats) / max(time.time() - t0, 1e-9)})
        if args.do_eval:
            results.update(squad.squad_scores(answers, args.predict_file))
    if rank == 0:
        with open(os.path.join(args.output_dir, "results.json"), "w") as f:
            json.dump(results, f, indent=1)
        print(json.dumps(results))
    if dist.is_initialized():
        dist.barrier()
        if own_group:
            dist.destroy_process_group()
    return results


if __name__ == "__main__":
    main()
