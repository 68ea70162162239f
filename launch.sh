#!/usr/bin/env bash
# Launch a script on all (or N) GPUs of this node, one process per GPU:  ./launch.sh [-n N] script.py [args...]
# Plays the role of the reference's scripts/launch.sh (torchrun wrapper + environment), without the NVSHMEM settings:
# the symmetric heap of this library is sized with TDB200_SYMM_HEAP_BYTES (default 4 GiB) and NVLS is switched with
# TDB200_NVLS=0|1.
set -euo pipefail
NPROC=""
if [[ "${1:-}" == "-n" ]]; then NPROC="$2"; shift 2; fi
if [[ -z "$NPROC" ]]; then NPROC=$(nvidia-smi -L 2>/dev/null | wc -l); fi
if [[ "$NPROC" -lt 1 ]]; then NPROC=1; fi
export CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-1}
export TDB200_SYMM_HEAP_BYTES=${TDB200_SYMM_HEAP_BYTES:-4294967296}
export PYTHONPATH="$(cd "$(dirname "$0")" && pwd):${PYTHONPATH:-}"
PORT=${MASTER_PORT:-$((20000 + RANDOM % 20000))}
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node="$NPROC" --master-addr 127.0.0.1 --master-port "$PORT" "$@"
