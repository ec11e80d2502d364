#!/bin/bash
# Runs a command (default: a shell) in the image with all or the named GPUs; results/ and the data directory
# are mounted from the host.  usage: launch.sh [command] [gpus, e.g. 0,1,2,3] [data directory]
set -euo pipefail
CMD="${1:-/bin/bash}"
DEVICES="${2:-all}"
DATA="${3:-$PWD/data}"
mkdir -p "$PWD/results"
docker run -it --rm --gpus "device=$DEVICES" --net=host --ipc=host --shm-size=1g \
    --ulimit memlock=-1 --ulimit stack=67108864 \
    -v "$PWD/results:/workspace/conef_b200/results" -v "$DATA:/workspace/data" \
    "${IMAGE:-conef_b200}" $CMD
