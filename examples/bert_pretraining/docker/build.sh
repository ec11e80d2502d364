#!/bin/bash
# Builds the image of examples/bert_pretraining/Dockerfile from the repository root.
set -euo pipefail
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../../.." && pwd)"
docker build --network=host --rm -f "$ROOT/examples/bert_pretraining/Dockerfile" -t "${IMAGE:-conef_b200}" "$ROOT"
