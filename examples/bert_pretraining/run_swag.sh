#!/bin/bash
# Fine-tune and/or evaluate on SWAG (counterpart of the reference's scripts/run_swag.sh: the same settings,
# as environment variables with defaults instead of eight positional arguments).
#
#   CHECKPOINT=results/bert/phase2/ckpt_1563.pt SWAG_DIR=data/swag VOCAB=vocab.txt examples/bert_pretraining/run_swag.sh
#
# MODE is "train eval" (default), "train" or "eval"; evaluation alone runs on one GPU.
set -euo pipefail

HERE=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
SWAG_DIR=${SWAG_DIR:-data/swag}
VOCAB=${VOCAB:-vocab.txt}
CONFIG=${CONFIG:-$HERE/configs/bert_large_config.json}
CHECKPOINT=${CHECKPOINT:-}
OUT=${OUT:-results/swag}
GPUS=${GPUS:-8}
BATCH=${BATCH:-12}
LR=${LR:-5e-6}
EPOCHS=${EPOCHS:-2}
MAX_STEPS=${MAX_STEPS:--1}
PRECISION=${PRECISION:-bf16}
MODE=${MODE:-train eval}
REDUCER=${REDUCER:-allreduce}
PYTHON=${PYTHON:-python}
DRY_RUN=${DRY_RUN:-0}

case "$MODE" in *train*) ;; *) GPUS=1 ;; esac
if [ "$GPUS" = "1" ]; then
  launcher=("$PYTHON")
else
  launcher=("$PYTHON" -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1
            --master-port "${MASTER_PORT:-29519}")
fi
args=(--data_dir "$SWAG_DIR" --vocab_file "$VOCAB" --config_file "$CONFIG" --output_dir "$OUT"
      --train_batch_size "$BATCH" --learning_rate "$LR" --num_train_epochs "$EPOCHS" --max_steps "$MAX_STEPS"
      --grad_reducer "$REDUCER")
case "$MODE" in *train*) args+=(--do_train) ;; esac
case "$MODE" in *eval*) args+=(--do_eval) ;; esac
[ -n "$CHECKPOINT" ] && args+=(--init_checkpoint "$CHECKPOINT")
[ "$PRECISION" = "bf16" ] && args+=(--bf16)

mkdir -p "$OUT"
if [ "$DRY_RUN" = "1" ]; then
  echo "${launcher[@]}" "$HERE/run_swag.py" "${args[@]}"
else
  "${launcher[@]}" "$HERE/run_swag.py" "${args[@]}" 2>&1 | tee "$OUT/logfile.txt"
fi
