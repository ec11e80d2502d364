#!/bin/bash
# Two-phase BERT pre-training (sequence length 128, then 512) on the GPUs of one node, with a
# compressed-gradient reducer.  The reference's launcher (scripts/run_pretraining_conef.sh) takes 28
# positional arguments and never passes --grad_reducer; this one takes named variables.
#
#   GPUS=8 REDUCER=conef_powersgd SHARDS128=/data/phase1 SHARDS512=/data/phase2 \
#       examples/bert_pretraining/run_pretraining.sh
# or with a hardware preset (configs/pretrain_config.sh):
#   PRESET=b200_8gpu_bf16_conef examples/bert_pretraining/run_pretraining.sh
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
if [[ -n "${PRESET:-}" ]]; then
    source "$HERE/configs/pretrain_config.sh"
    "$PRESET"
fi
GPUS="${GPUS:-8}"
REDUCER="${REDUCER:-conef_powersgd}"
CONFIG="${CONFIG:-$HERE/configs/bert_large_config.json}"
OUT="${OUT:-results/bert}"
BATCH1="${BATCH1:-64}";  STEPS1="${STEPS1:-7038}";  LR1="${LR1:-6e-3}";  ACCUM1="${ACCUM1:-1}"
BATCH2="${BATCH2:-8}";   STEPS2="${STEPS2:-1563}";  LR2="${LR2:-4e-3}";  ACCUM2="${ACCUM2:-1}"
# --train_batch_size is per process and per optimizer step: micro-batch x accumulation steps
TBS1=$((BATCH1 * ACCUM1)); TBS2=$((BATCH2 * ACCUM2))
PORT="${PORT:-29500}"
MODEL_ARGS=(--config_file "$CONFIG")
if [[ -n "${MODEL:-}" ]]; then MODEL_ARGS=(--bert_model "$MODEL"); fi
EXTRA=()
if [[ -n "${POST_ACCUMULATION:-}" ]]; then EXTRA+=(--allreduce_post_accumulation); fi
if [[ -n "${POST_ACCUMULATION_FP16:-}" ]]; then EXTRA+=(--allreduce_post_accumulation_fp16); fi
COMMON=("${MODEL_ARGS[@]}" "${EXTRA[@]}" --seed "${SEED:-42}" --compression_ratio "${RATIO:-0.1}" --grad_reducer "$REDUCER" --matrix_approximation_rank "${RANK_R:-8}"
        --sketch_size "${SKETCH:-0.1}" --beta "${BETA:-0.9}" --start_compression_percentage "${START:-0.1}"
        --num_steps_per_checkpoint "${CKPT_EVERY:-200}")
launch() { python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 \
               --master-port "$PORT" "$HERE/run_pretraining.py" "$@"; }

# phase 1: sequence length 128, 20 predictions per sequence
launch "${COMMON[@]}" --output_dir "$OUT/phase1" --max_seq_length 128 --max_predictions_per_seq 20 \
       --train_batch_size "$TBS1" --gradient_accumulation_steps "$ACCUM1" --max_steps "$STEPS1" \
       --learning_rate "$LR1" --warmup_proportion "${WARMUP1:-0.2843}" \
       ${SHARDS128:+--input_dir "$SHARDS128"} --resume_from_checkpoint
# phase 2: sequence length 512, 80 predictions per sequence, from the weights of phase 1 (a new run:
# optimizer, schedule and reducer state start fresh)
launch "${COMMON[@]}" --output_dir "$OUT/phase2" --max_seq_length 512 --max_predictions_per_seq 80 \
       --train_batch_size "$TBS2" --gradient_accumulation_steps "$ACCUM2" --max_steps "$STEPS2" \
       --learning_rate "$LR2" --warmup_proportion "${WARMUP2:-0.128}" \
       ${SHARDS512:+--input_dir "$SHARDS512"} --resume_from_checkpoint --init_checkpoint "$OUT/phase1"
