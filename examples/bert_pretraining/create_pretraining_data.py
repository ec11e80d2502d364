"""Text -> masked-LM / next-sentence instances -> shard files for ``run_pretraining.py --input_dir``.

Input: one sentence per line, blank lines between documents (the format of the reference's
``create_pretraining_data.py``).  Output: ``<output_prefix>_<k>.npz`` shards.

    python examples/bert_pretraining/create_pretraining_data.py --input_file corpus.txt \
        --vocab_file vocab.txt --output_prefix shards/part --max_seq_length 128 --shards 4
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from conef_b200.data.pretraining import (create_training_instances, instances_to_arrays, read_documents,  # noqa: E402
                                         write_shard)
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--input_file", required=True, help="comma-separated text files")
    p.add_argument("--vocab_file", required=True)
    p.add_argument("--output_prefix", required=True)
    p.add_argument("--shards", type=int, default=1)
    p.add_argument("--do_lower_case", action="store_true", default=True)
    p.add_argument("--max_seq_length", type=int, default=128)
    p.add_argument("--max_predictions_per_seq", type=int, default=20)
    p.add_argument("--masked_lm_prob", type=float, default=0.15)
    p.add_argument("--short_seq_prob", type=float, default=0.1)
    p.add_argument("--dupe_factor", type=int, default=5)
    p.add_argument("--random_seed", type=int, default=12345)
    args = p.parse_args()

    tok = BertTokenizer(args.vocab_file, do_lower_case=args.do_lower_case)
    docs = read_documents(args.input_file.split(","), tok)
    inst = create_training_instances(docs, list(tok.vocab.keys()), args.max_seq_length, args.dupe_factor,
                                     args.short_seq_prob, args.masked_lm_prob, args.max_predictions_per_seq,
                                     args.random_seed)
    os.makedirs(os.path.dirname(os.path.abspath(args.output_prefix)), exist_ok=True)
    per = (len(inst) + args.shards - 1) // args.shards
    for k in range(args.shards):
        part = inst[k * per : (k + 1) * per]
        if not part:
            break
        path = f"{args.output_prefix}_{k}.npz"
        write_shard(path, instances_to_arrays(part, tok, args.max_seq_length, args.max_predictions_per_seq))
        print(f"{path}: {len(part)} instances")


if __name__ == "__main__":
    main()
