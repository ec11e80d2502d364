#!/bin/bash
# Start a Triton Inference Server container on the model repository written by export.py.
# (Counterpart of the reference's examples/BertPretraining/triton/launch_triton_server.sh.)
#
#   REPOSITORY=/models/repo GPUS=0 IMAGE=nvcr.io/nvidia/tritonserver:25.01-py3 bash launch_server.sh
#
# Needs a container runtime with GPU support; nothing else in this folder does.
set -euo pipefail

REPOSITORY=${REPOSITORY:-$PWD/results/model_repository}
GPUS=${GPUS:-all}
IMAGE=${IMAGE:-nvcr.io/nvidia/tritonserver:25.01-py3}
NAME=${NAME:-conef_triton_server}
HTTP_PORT=${HTTP_PORT:-8000}
GRPC_PORT=${GRPC_PORT:-8001}
METRICS_PORT=${METRICS_PORT:-8002}
DRY_RUN=${DRY_RUN:-0}

if [ "$GPUS" = "all" ]; then GPU_FLAG="all"; else GPU_FLAG="device=${GPUS}"; fi

cmd=(docker run -d --rm
     --gpus "$GPU_FLAG"
     --shm-size=1g --ulimit memlock=-1 --ulimit stack=67108864
     -p "${HTTP_PORT}:8000" -p "${GRPC_PORT}:8001" -p "${METRICS_PORT}:8002"
     --name "$NAME"
     -v "${REPOSITORY}:/models:ro"
     "$IMAGE" tritonserver --model-repository=/models --strict-model-config=true)

if [ "$DRY_RUN" = "1" ]; then
  echo "${cmd[@]}"
else
  "${cmd[@]}"
fi
