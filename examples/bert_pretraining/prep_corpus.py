#!/usr/bin/env python
"""Corpus preparation pipeline for BERT pre-training, from local files.

Counterpart of the reference's ``examples/BertPretraining/data/bertPrep.py``: one ``--action`` per call.

    text_formatting          raw corpus -> one article per line   (--dataset wikicorpus_en | bookscorpus)
    sharding                 formatted corpora -> sentence-per-line training / test shards
    create_pretraining_files shards -> masked-LM / next-sentence instances (.npz) for run_pretraining.py --input_dir
    download                 not available: the machines this runs on have no network; place the raw
                             corpus under <working_dir>/download/<dataset> yourself

    python examples/bert_pretraining/prep_corpus.py --action text_formatting --dataset bookscorpus --working_dir data
    python examples/bert_pretraining/prep_corpus.py --action sharding --dataset bookscorpus --working_dir data \
        --n_training_shards 8 --n_test_shards 2 --fraction_test_set 0.1
    python examples/bert_pretraining/prep_corpus.py --action create_pretraining_files --dataset bookscorpus \
        --working_dir data --vocab_file vocab.txt --max_seq_length 128
"""
import argparse
import glob
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from conef_b200.data import corpus_prep  # noqa: E402
from conef_b200.data.pretraining import (create_training_instances, instances_to_arrays, read_documents,  # noqa: E402
                                         write_shard)
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402

DATASETS = ("bookscorpus", "wikicorpus_en", "wikicorpus_zh", "books_wiki_en_corpus")


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--action", required=True,
                   choices=["download", "text_formatting", "sharding", "create_pretraining_files"])
    p.add_argument("--dataset", required=True, choices=DATASETS)
    p.add_argument("--working_dir", default=os.environ.get("BERT_PREP_WORKING_DIR", "data"))
    p.add_argument("--input_files", default=None, help="comma-separated formatted files (default: the dataset's)")
    p.add_argument("--n_training_shards", type=int, default=256)
    p.add_argument("--n_test_shards", type=int, default=256)
    p.add_argument("--fraction_test_set", type=float, default=0.1)
    p.add_argument("--vocab_file", default=None)
    p.add_argument("--do_lower_case", type=int, default=1)
    p.add_argument("--max_seq_length", type=int, default=512)
    p.add_argument("--max_predictions_per_seq", type=int, default=20)
    p.add_argument("--masked_lm_prob", type=float, default=0.15)
    p.add_argument("--short_seq_prob", type=float, default=0.1)
    p.add_argument("--dupe_factor", type=int, default=5)
    p.add_argument("--random_seed", type=int, default=12345)
    args = p.parse_args()

    wd = args.working_dir
    folder = {k: os.path.join(wd, k) for k in ("download", "formatted_one_article_per_line", "sharded", "npz")}
    one_line = lambda name: os.path.join(folder["formatted_one_article_per_line"], f"{name}_one_article_per_line.txt")
    parts = ["bookscorpus", "wikicorpus_en"] if args.dataset == "books_wiki_en_corpus" else [args.dataset]
    shard_tag = f"{args.dataset}/training_shards_{args.n_training_shards}_test_shards_{args.n_test_shards}" \
                f"_fraction_{args.fraction_test_set}"

    if args.action == "download":
        sys.exit("download: not available offline; put the raw corpus under "
                 f"{os.path.join(folder['download'], args.dataset)} and continue with --action text_formatting")

    if args.action == "text_formatting":
        os.makedirs(folder["formatted_one_article_per_line"], exist_ok=True)
        for name in parts:
            src = os.path.join(folder["download"], name)
            fmt = corpus_prep.format_bookscorpus if name == "bookscorpus" else corpus_prep.format_wikicorpus
            n = fmt(src, one_line(name))
            print(f"{name}: {n} articles -> {one_line(name)}")
        return

    if args.action == "sharding":
        inputs = args.input_files.split(",") if args.input_files else [one_line(name) for name in parts]
        prefix = os.path.join(folder["sharded"], shard_tag, args.dataset)
        sh = corpus_prep.Sharding(inputs, prefix, args.n_training_shards, args.n_test_shards, args.fraction_test_set)
        sh.load_articles()
        sh.segment_articles_into_sentences()
        sh.distribute_articles_over_shards()
        for name in sh.write_shards_to_disk():
            print(name)
        return

    if not args.vocab_file:
        sys.exit("create_pretraining_files needs --vocab_file")
    tok = BertTokenizer(args.vocab_file, do_lower_case=bool(args.do_lower_case))
    out_dir = os.path.join(folder["npz"], shard_tag, f"seq_{args.max_seq_length}_pred_{args.max_predictions_per_seq}")
    os.makedirs(out_dir, exist_ok=True)
    shards = sorted(glob.glob(os.path.join(folder["sharded"], shard_tag, "*.txt")))
    if not shards:
        sys.exit(f"no shards under {os.path.join(folder['sharded'], shard_tag)}: run --action sharding first")
    for path in shards:
        docs = read_documents([path], tok)
        inst = create_training_instances(docs, list(tok.vocab.keys()), args.max_seq_length, args.dupe_factor,
                                         args.short_seq_prob, args.masked_lm_prob, args.max_predictions_per_seq,
                                         args.random_seed)
        arrays = instances_to_arrays(inst, tok, args.max_seq_length, args.max_predictions_per_seq)
        out = os.path.join(out_dir, os.path.basename(path).replace(".txt", ".npz"))
        write_shard(out, arrays)
        print(f"{out}: {len(inst)} instances")


if __name__ == "__main__":
    main()
