#!/usr/bin/env bash
# Two-rank tensor-parallel smoke run of scripts/smoke_train.py on one node (reference: scripts/smoke_train_dist.sh).
# NCCL on GPUs, Gloo on a CPU-only machine; rendezvous on 127.0.0.1.
set -euo pipefail
cd "$(dirname "$0")/.."
NPROC="${NPROC:-2}"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NPROC" --master-addr 127.0.0.1 \
     --master-port "${MASTER_PORT:-29517}" scripts/smoke_train.py "$@"
