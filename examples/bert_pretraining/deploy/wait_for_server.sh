#!/bin/bash
# Block until the server answers its liveness and readiness probes, or give up after LIMIT seconds.
# (Counterpart of the reference's examples/BertPretraining/triton/wait_for_triton_server.sh, which
# loops without a limit.)
#
#   bash wait_for_server.sh [host[:port]] [limit_seconds]
set -uo pipefail

SERVER=${1:-127.0.0.1:8000}
LIMIT=${2:-120}
case "$SERVER" in *:*) ;; *) SERVER="$SERVER:8000" ;; esac

probe() { curl -m 1 -L -s -o /dev/null -w '%{http_code}' "http://$SERVER/v2/health/$1" 2>/dev/null || true; }

echo "waiting for the inference server at http://$SERVER (at most ${LIMIT}s)"
for ((i = 0; i < LIMIT; i++)); do
  if [ "$(probe live)" = "200" ] && [ "$(probe ready)" = "200" ]; then
    echo "server is ready"
    exit 0
  fi
  sleep 1
done
echo "server did not become ready within ${LIMIT}s" >&2
exit 1
