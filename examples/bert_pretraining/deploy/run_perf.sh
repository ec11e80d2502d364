#!/bin/bash
# Sequences per second of the exported model over a sweep of batch sizes, as CSV.
# (Counterpart of the reference's examples/BertPretraining/triton/run_perf_client.sh and
# generate_figures.sh, whose figures are plots of this table.)
#
#   REPOSITORY=/models MODEL_NAME=bert_qa bash run_perf.sh [batch sizes...]        # in-process
#   TRITON_URL=127.0.0.1:8000 MODEL_NAME=bert_qa bash run_perf.sh 1 2 4 8          # through a server
set -euo pipefail

HERE=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
MODEL_NAME=${MODEL_NAME:-bert_qa}
SEQ_LENGTH=${SEQ_LENGTH:-384}
ITERS=${ITERS:-20}
OUT=${OUT:-perf_${MODEL_NAME}.csv}
PYTHON=${PYTHON:-python}
if [ -n "${TRITON_URL:-}" ]; then where=(--triton_url "$TRITON_URL"); else where=(--local_repository "${REPOSITORY:-$PWD/results/model_repository}"); fi
[ "$#" -gt 0 ] || set -- 1 2 4 8

echo "batch_size,seq_length,seq_per_s,ms_per_request" > "$OUT"
for b in "$@"; do
  "$PYTHON" "$HERE/client.py" "${where[@]}" --model_name "$MODEL_NAME" --perf --batch_size "$b" \
      --max_seq_length "$SEQ_LENGTH" --perf_iters "$ITERS" ${PERF_VOCAB:+--perf_vocab "$PERF_VOCAB"} ${DEVICE:+--device "$DEVICE"} \
    | "$PYTHON" -c 'import json,sys; d=json.loads(sys.stdin.read().strip().splitlines()[-1]); print("%d,%d,%.2f,%.3f" % (d["batch_size"], d["seq_length"], d["seq_per_s"], d["ms_per_request"]))' >> "$OUT"
done
cat "$OUT"
