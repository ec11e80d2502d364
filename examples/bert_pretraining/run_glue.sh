#!/bin/bash
# Fine-tune and/or evaluate on a GLUE task (counterpart of the reference's scripts/run_glue.sh: the same
# settings, as environment variables with defaults instead of sixteen positional arguments).
#
#   source examples/bert_pretraining/configs/glue_config.sh && glue_mrpc && b200_8gpu_bf16
#   CHECKPOINT=results/bert/phase2/ckpt_1563.pt DATA_DIR=glue/MRPC VOCAB=vocab.txt examples/bert_pretraining/run_glue.sh
#
# MODE is "train eval" (default), "train" or "eval"; evaluation alone runs on one GPU.
set -euo pipefail

HERE=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
TASK=${TASK:-mrpc}
DATA_DIR=${DATA_DIR:-data/glue/MRPC}
VOCAB=${VOCAB:-vocab.txt}
CONFIG=${CONFIG:-$HERE/configs/bert_large_config.json}
CHECKPOINT=${CHECKPOINT:-}
OUT=${OUT:-results/glue/$TASK}
GPUS=${GPUS:-8}
BATCH=${BATCH:-16}
ACCUM=${ACCUM:-1}
LR=${LR:-2.4e-5}
WARMUP=${WARMUP:-0.1}
EPOCHS=${EPOCHS:-3}
MAX_STEPS=${MAX_STEPS:--1}
PRECISION=${PRECISION:-bf16}
SEED=${SEED:-2}
MODE=${MODE:-train eval}
REDUCER=${REDUCER:-allreduce}
PYTHON=${PYTHON:-python}
DRY_RUN=${DRY_RUN:-0}

case "$MODE" in *train*) ;; *) GPUS=1 ;; esac

if [ "$GPUS" = "1" ]; then
  launcher=("$PYTHON")
else
  launcher=("$PYTHON" -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1
            --master-port "${MASTER_PORT:-29517}")
fi

args=(--task_name "$TASK" --data_dir "$DATA_DIR" --vocab_file "$VOCAB" --config_file "$CONFIG" --output_dir "$OUT"
      --train_batch_size "$BATCH" --gradient_accumulation_steps "$ACCUM" --learning_rate "$LR"
      --warmup_proportion "$WARMUP" --num_train_epochs "$EPOCHS" --max_steps "$MAX_STEPS" --seed "$SEED"
      --grad_reducer "$REDUCER")
case "$MODE" in *train*) args+=(--do_train) ;; esac
case "$MODE" in *eval*) args+=(--do_eval) ;; esac
[ -n "$CHECKPOINT" ] && args+=(--init_checkpoint "$CHECKPOINT")
[ "$PRECISION" = "bf16" ] && args+=(--bf16)

mkdir -p "$OUT"
if [ "$DRY_RUN" = "1" ]; then
  echo "${launcher[@]}" "$HERE/run_glue.py" "${args[@]}"
else
  "${launcher[@]}" "$HERE/run_glue.py" "${args[@]}" 2>&1 | tee "$OUT/logfile.txt"
fi
