#!/bin/bash
# Export a fine-tuned question-answering checkpoint into a model repository and check it in-process.
# (Counterpart of the reference's examples/BertPretraining/triton/export_model.sh and evaluate.sh.)
#
#   bash export_model.sh <checkpoint> [batch_size] [precision fp16|fp32] [format ts-trace|onnx] [seq_length]
#
# Environment: BERT_MODEL (base|large|tiny), CONFIG_FILE, REPOSITORY, MODEL_NAME, VOCAB_FILE and SQUAD_FILE
# (both optional: with them the exported model answers the file and prints exact match and F1).
set -euo pipefail

HERE=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
CHECKPOINT=${1:-}
BATCH_SIZE=${2:-8}
PRECISION=${3:-fp16}
FORMAT=${4:-ts-trace}
SEQ_LENGTH=${5:-384}
BERT_MODEL=${BERT_MODEL:-large}
REPOSITORY=${REPOSITORY:-$PWD/results/model_repository}
MODEL_NAME=${MODEL_NAME:-bert_qa_${FORMAT//-/_}}
PYTHON=${PYTHON:-python}
DRY_RUN=${DRY_RUN:-0}

args=(--repository "$REPOSITORY" --model_name "$MODEL_NAME" --format "$FORMAT" --bert_model "$BERT_MODEL"
      --max_seq_length "$SEQ_LENGTH" --batch_size "$BATCH_SIZE" --tolerance 0.05)
[ -n "$CHECKPOINT" ] && args+=(--init_checkpoint "$CHECKPOINT")
[ -n "${CONFIG_FILE:-}" ] && args+=(--config_file "$CONFIG_FILE")
[ "$PRECISION" = "fp16" ] && args+=(--fp16)

run() { if [ "$DRY_RUN" = "1" ]; then echo "$@"; else "$@"; fi; }

run "$PYTHON" "$HERE/export.py" "${args[@]}"
if [ -n "${VOCAB_FILE:-}" ] && [ -n "${SQUAD_FILE:-}" ]; then
  run "$PYTHON" "$HERE/client.py" --local_repository "$REPOSITORY" --model_name "$MODEL_NAME" --vocab_file "$VOCAB_FILE" \
      --squad_file "$SQUAD_FILE" --evaluate --batch_size "$BATCH_SIZE" --max_seq_length "$SEQ_LENGTH" \
      --output_file "$REPOSITORY/$MODEL_NAME/predictions.json"
fi
run "$PYTHON" "$HERE/client.py" --local_repository "$REPOSITORY" --model_name "$MODEL_NAME" --perf \
    --batch_size "$BATCH_SIZE" --max_seq_length "$SEQ_LENGTH"
