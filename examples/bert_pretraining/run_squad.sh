#!/bin/bash
# Fine-tune on SQuAD and/or predict and score (counterpart of the reference's scripts/run_squad.sh: the same
# settings, as environment variables with defaults instead of thirteen positional arguments).
#
#   source examples/bert_pretraining/configs/squad_config.sh && squad_b200_8gpu_bf16
#   CHECKPOINT=results/bert/phase2/ckpt_1563.pt SQUAD_DIR=squad/v1.1 VOCAB=vocab.txt examples/bert_pretraining/run_squad.sh
#
# MODE is "train eval" (default), "train", "eval" (predict and score) or "prediction" (predict only);
# SQUAD_DIR holds train-v1.1.json / dev-v1.1.json, or the v2.0 files with VERSION=2.0.
set -euo pipefail

HERE=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
SQUAD_DIR=${SQUAD_DIR:-data/squad/v1.1}
VERSION=${VERSION:-1.1}
VOCAB=${VOCAB:-vocab.txt}
CONFIG=${CONFIG:-$HERE/configs/bert_large_config.json}
CHECKPOINT=${CHECKPOINT:-}
OUT=${OUT:-results/squad}
GPUS=${GPUS:-8}
BATCH=${BATCH:-4}
ACCUM=${ACCUM:-1}
LR=${LR:-3e-5}
WARMUP=${WARMUP:-0.1}
EPOCHS=${EPOCHS:-2.0}
MAX_STEPS=${MAX_STEPS:--1}
PRECISION=${PRECISION:-bf16}
SEED=${SEED:-1}
MODE=${MODE:-train eval}
REDUCER=${REDUCER:-allreduce}
PYTHON=${PYTHON:-python}
DRY_RUN=${DRY_RUN:-0}

case "$MODE" in *train*) ;; *) GPUS=1 ;; esac

if [ "$GPUS" = "1" ]; then
  launcher=("$PYTHON")
else
  launcher=("$PYTHON" -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1
            --master-port "${MASTER_PORT:-29518}")
fi

args=(--vocab_file "$VOCAB" --config_file "$CONFIG" --output_dir "$OUT" --train_batch_size "$BATCH"
      --gradient_accumulation_steps "$ACCUM" --learning_rate "$LR" --warmup_proportion "$WARMUP"
      --num_train_epochs "$EPOCHS" --max_steps "$MAX_STEPS" --seed "$SEED" --grad_reducer "$REDUCER"
      --max_seq_length 384 --doc_stride 128)
case "$MODE" in *train*) args+=(--do_train --train_file "$SQUAD_DIR/train-v$VERSION.json") ;; esac
case "$MODE" in *eval*) args+=(--do_predict --do_eval --predict_file "$SQUAD_DIR/dev-v$VERSION.json") ;; esac
case "$MODE" in *prediction*) args+=(--do_predict --predict_file "$SQUAD_DIR/dev-v$VERSION.json") ;; esac
[ "$VERSION" = "2.0" ] && args+=(--version_2_with_negative)
[ -n "$CHECKPOINT" ] && args+=(--init_checkpoint "$CHECKPOINT")
[ "$PRECISION" = "bf16" ] && args+=(--bf16)

mkdir -p "$OUT"
if [ "$DRY_RUN" = "1" ]; then
  echo "${launcher[@]}" "$HERE/run_squad.py" "${args[@]}"
else
  "${launcher[@]}" "$HERE/run_squad.py" "${args[@]}" 2>&1 | tee "$OUT/logfile.txt"
fi
