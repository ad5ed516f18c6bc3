#!/bin/bash
# Launch a script with one process per GPU of this node:
#   ./launch.sh [--nproc N] script.py [args...]
# (reference: launch.sh, which also sets NVSHMEM variables that have no counterpart here)
NPROC=${NPROC:-$(nvidia-smi -L 2>/dev/null | wc -l)}
if [ "$1" = "--nproc" ]; then NPROC=$2; shift 2; fi
[ "${NPROC:-0}" -ge 1 ] || NPROC=1
export CUDA_MODULE_LOADING=${CUDA_MODULE_LOADING:-LAZY}
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NPROC" \
  --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29500}" "$@"
