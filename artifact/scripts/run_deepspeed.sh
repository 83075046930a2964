#!/usr/bin/env bash
# DeepSpeed baseline for one experiment on this node.
#   artifact/scripts/run_deepspeed.sh --gpus 8 --model qwen3_1b --pp 4 --dp 2 --zero-stage 1 [--steps N] ...
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
gpus=8
args=()
while (($#)); do
  case "$1" in
    --gpus) gpus="$2"; shift 2 ;;
    *) args+=("$1"); shift ;;
  esac
done
if ! command -v deepspeed >/dev/null 2>&1; then
  echo "run_deepspeed.sh: the deepspeed launcher is not installed" >&2
  exit 3
fi
exec deepspeed --num_gpus="$gpus" --master_addr 127.0.0.1 "$HERE/../run_deepspeed.py" "${args[@]}"
