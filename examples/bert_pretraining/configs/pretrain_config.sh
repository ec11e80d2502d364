#!/bin/bash
# Hardware presets for run_pretraining.sh: one shell function per machine shape, each setting the
# variables that launcher reads.  The reference ships the same idea for DGX A100 / DGX-2 / DGX-1 x
# fp16 / tf32 / fp32 (scripts/configs/pretrain_config.sh:16-252); these are for B200 nodes, bf16
# autocast, with the per-GPU batch sized for 180 GB of HBM3e (BERT-large, sequence length 128: 64
# sequences per GPU and micro-batch fit without activation checkpointing; length 512: 16).
#
#   source examples/bert_pretraining/configs/pretrain_config.sh && b200_8gpu_bf16_conef
#   examples/bert_pretraining/run_pretraining.sh
#
# Global batch = GPUS x BATCH x ACCUM.  The LAMB recipe of the reference uses a global batch of
# 8192 (phase 1) and 4096 (phase 2): 8 x 64 x 16 and 8 x 16 x 32.

_b200_common () {
    export CONFIG="${CONFIG:-$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/bert_large_config.json}"
    export STEPS1=7038 LR1=6e-3 WARMUP1=0.2843
    export STEPS2=1563 LR2=4e-3 WARMUP2=0.128
    export CKPT_EVERY=200 SEED=42
}

# ---- one node, eight GPUs -----------------------------------------------------------------------
b200_8gpu_bf16_conef () {            # PowerSGD rank 8 + count-sketch error memory (10 % of the gradient)
    _b200_common
    export GPUS=8 REDUCER=conef_powersgd RANK_R=8 SKETCH=0.1 BETA=0.9 START=0.1
    export BATCH1=64 ACCUM1=16 BATCH2=16 ACCUM2=32
}

b200_8gpu_bf16_ef () {               # PowerSGD rank 8 + dense error feedback
    b200_8gpu_bf16_conef
    export REDUCER=ef_powersgd
}

b200_8gpu_bf16_randomblock () {      # random contiguous blocks (10 %) + count-sketch error memory
    b200_8gpu_bf16_conef
    export REDUCER=conef_randomblock RATIO=0.1
}

b200_8gpu_bf16_allreduce () {        # uncompressed DDP, the comparison line
    b200_8gpu_bf16_conef
    export REDUCER=allreduce
}

b200_8gpu_bf16_post_accumulation () {   # no DDP: one fp16 all-reduce of all gradients per optimizer step
    b200_8gpu_bf16_conef
    export REDUCER=allreduce POST_ACCUMULATION=1 POST_ACCUMULATION_FP16=1
}

# ---- smaller shapes -------------------------------------------------------------------------------
b200_4gpu_bf16_conef () { b200_8gpu_bf16_conef; export GPUS=4 ACCUM1=32 ACCUM2=64; }
b200_2gpu_bf16_conef () { b200_8gpu_bf16_conef; export GPUS=2 ACCUM1=64 ACCUM2=128; }
b200_1gpu_bf16_conef () { b200_8gpu_bf16_conef; export GPUS=1 ACCUM1=128 ACCUM2=256; }

# ---- a functional check that finishes in a minute on any machine (tiny model, synthetic shards) ----
smoke_1gpu () {
    export GPUS=1 REDUCER=conef_powersgd RANK_R=2 SKETCH=0.1 BETA=0.9 START=0.1 MODEL=tiny
    export BATCH1=8 ACCUM1=1 STEPS1=6 LR1=1e-3 WARMUP1=0.1 BATCH2=4 ACCUM2=1 STEPS2=4 LR2=1e-3 WARMUP2=0.1
    export CKPT_EVERY=100 SEED=42
}

if [[ "${BASH_SOURCE[0]}" == "$0" ]]; then      # run as a script: print what a preset sets
    "${1:?usage: pretrain_config.sh <preset>}"
    env | grep -E '^(GPUS|REDUCER|RANK_R|SKETCH|BETA|START|RATIO|BATCH[12]|ACCUM[12]|STEPS[12]|LR[12]|WARMUP[12]|CKPT_EVERY|SEED|MODEL|POST_ACCUMULATION(_FP16)?)=' | sort
fi
