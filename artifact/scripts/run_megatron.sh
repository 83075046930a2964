#!/usr/bin/env bash
# Megatron-LM baseline for one experiment: forwards its arguments to artifact/run_megatron.py on this node.
#   MEGATRON_HOME=/path/to/Megatron-LM artifact/scripts/run_megatron.sh --model qwen3_9b --pp 4 --dp 2 \
#       --nnodes 1 --nproc-per-node 8 [--micro-bs N] [--global-bs N] [--seq-length N] [--train-iters N]
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
exec "${PYTHON:-python}" "$HERE/../run_megatron.py" "$@"
