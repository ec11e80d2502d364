#!/bin/bash
# Task and machine presets for run_glue.sh: a task function, then a machine function.  The reference ships
# the same idea for MRPC and SST-2 on DGX A100 / DGX-2 / DGX-1 (scripts/configs/glue_config.sh); these are
# for B200 nodes with bf16 autocast.  The per-GPU batch follows from the task's global batch, the number of
# GPUs and what one GPU takes per micro-batch (CAPACITY); the rest becomes gradient accumulation.
#
#   source examples/bert_pretraining/configs/glue_config.sh && glue_mrpc && b200_8gpu_bf16
#   examples/bert_pretraining/run_glue.sh

_glue_split_batch () {               # GLOBAL_BATCH, GPUS, CAPACITY -> BATCH (per GPU and step), ACCUM
    export BATCH=$((GLOBAL_BATCH / GPUS))
    [ "$BATCH" -ge 1 ] || export BATCH=1
    export ACCUM=1
    while [ $((BATCH / ACCUM)) -gt "$CAPACITY" ]; do export ACCUM=$((ACCUM * 2)); done
}

glue_mrpc ()  { export TASK=mrpc  GLOBAL_BATCH=128 LR=2.4e-5 WARMUP=0.1 EPOCHS=3; }
glue_sst2 ()  { export TASK=sst-2 GLOBAL_BATCH=256 LR=2.4e-5 WARMUP=0.1 EPOCHS=3; }
glue_cola ()  { export TASK=cola  GLOBAL_BATCH=128 LR=2.4e-5 WARMUP=0.1 EPOCHS=3; }
glue_mnli ()  { export TASK=mnli  GLOBAL_BATCH=256 LR=2.4e-5 WARMUP=0.1 EPOCHS=3; }

b200_8gpu_bf16 () { export GPUS=8 CAPACITY=256 PRECISION=bf16; _glue_split_batch; }
b200_4gpu_bf16 () { export GPUS=4 CAPACITY=256 PRECISION=bf16; _glue_split_batch; }
b200_1gpu_bf16 () { export GPUS=1 CAPACITY=256 PRECISION=bf16; _glue_split_batch; }
b200_1gpu_fp32 () { export GPUS=1 CAPACITY=64  PRECISION=fp32; _glue_split_batch; }

glue_show () {
    echo "TASK=$TASK GPUS=$GPUS BATCH=$BATCH ACCUM=$ACCUM LR=$LR WARMUP=$WARMUP EPOCHS=$EPOCHS PRECISION=$PRECISION"
}
