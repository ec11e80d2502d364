#!/bin/bash
# From a raw corpus on disk to the two sets of pre-training shards (sequence length 128 for phase 1, 512 for
# phase 2).  Counterpart of the reference's examples/BertPretraining/data/create_datasets_from_start.sh without
# its download steps (no network): put the raw corpus under $WORKING_DIR/download/<dataset> first.
#
#   WORKING_DIR=data VOCAB=vocab.txt bash examples/bert_pretraining/create_datasets.sh [wiki_only | wiki_books | books_only]
#
# SHARDS_TRAIN / SHARDS_TEST / TEST_FRACTION size the sharding step; DRY_RUN=1 prints the commands.
set -euo pipefail

HERE=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
WHAT=${1:-wiki_only}
WORKING_DIR=${WORKING_DIR:-${BERT_PREP_WORKING_DIR:-data}}
VOCAB=${VOCAB:-vocab.txt}
SHARDS_TRAIN=${SHARDS_TRAIN:-256}
SHARDS_TEST=${SHARDS_TEST:-256}
TEST_FRACTION=${TEST_FRACTION:-0.1}
PYTHON=${PYTHON:-python}
DRY_RUN=${DRY_RUN:-0}

case "$WHAT" in
  wiki_only)  FORMAT=(wikicorpus_en); DATASET=wikicorpus_en ;;
  books_only) FORMAT=(bookscorpus); DATASET=bookscorpus ;;
  wiki_books) FORMAT=(bookscorpus wikicorpus_en); DATASET=books_wiki_en_corpus ;;
  *) echo "usage: $0 [wiki_only | wiki_books | books_only]" >&2; exit 2 ;;
esac

prep() {
  if [ "$DRY_RUN" = "1" ]; then echo "$PYTHON" "$HERE/prep_corpus.py" --working_dir "$WORKING_DIR" "$@"
  else "$PYTHON" "$HERE/prep_corpus.py" --working_dir "$WORKING_DIR" "$@"; fi
}
shards=(--n_training_shards "$SHARDS_TRAIN" --n_test_shards "$SHARDS_TEST" --fraction_test_set "$TEST_FRACTION")

for d in "${FORMAT[@]}"; do prep --action text_formatting --dataset "$d"; done
prep --action sharding --dataset "$DATASET" "${shards[@]}"
prep --action create_pretraining_files --dataset "$DATASET" "${shards[@]}" --vocab_file "$VOCAB" --do_lower_case 1 \
     --max_seq_length 128 --max_predictions_per_seq 20
prep --action create_pretraining_files --dataset "$DATASET" "${shards[@]}" --vocab_file "$VOCAB" --do_lower_case 1 \
     --max_seq_length 512 --max_predictions_per_seq 80
