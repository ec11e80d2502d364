#!/bin/bash
# Machine presets for run_squad.sh (the reference ships them for DGX A100 / DGX-2 / DGX-1,
# scripts/configs/squad_config.sh): B200 nodes, bf16 autocast.  BATCH is windows of 384 tokens per GPU and
# optimizer step; the recipe's global batch is 32.
#
#   source examples/bert_pretraining/configs/squad_config.sh && squad_b200_8gpu_bf16
#   CHECKPOINT=... SQUAD_DIR=squad/v1.1 VOCAB=vocab.txt examples/bert_pretraining/run_squad.sh

_squad_common () { export EPOCHS=2.0 LR=3e-5 WARMUP=0.1 SEED=1 MAX_STEPS=-1; }

squad_b200_8gpu_bf16 () { _squad_common; export GPUS=8 BATCH=4  ACCUM=1 PRECISION=bf16; }
squad_b200_4gpu_bf16 () { _squad_common; export GPUS=4 BATCH=8  ACCUM=1 PRECISION=bf16; }
squad_b200_1gpu_bf16 () { _squad_common; export GPUS=1 BATCH=32 ACCUM=1 PRECISION=bf16; }
squad_b200_1gpu_fp32 () { _squad_common; export GPUS=1 BATCH=32 ACCUM=2 PRECISION=fp32; }
squad_b200_8gpu_bf16_conef () { squad_b200_8gpu_bf16; export REDUCER=conef_powersgd; }
