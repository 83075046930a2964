#!/usr/bin/env bash
# TorchTitan baseline for one experiment on this node (Qwen3 MoE flavours of torchtitan.models.qwen3).
#   artifact/scripts/run_torchtitan.sh --gpus 8 --flavor 9B --pp 4 --dp 2 [--ep N] [--seq-len N] [--batch N]
#       [--steps N] [--bmm-experts]
# --bmm-experts sets TORCHTITAN_USE_BMM_EXPERTS=1 and puts artifact/ on PYTHONPATH so that sitecustomize.py
# swaps TorchTitan's grouped-expert forward for the padded batched-matmul form the reference compared against.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
gpus=8; flavor=9B; pp=1; dp=1; ep=1; seq=512; batch=4; steps=10; bmm=0
while (($#)); do
  case "$1" in
    --gpus) gpus="$2"; shift 2 ;;
    --flavor|--model) flavor="$2"; shift 2 ;;
    --pp) pp="$2"; shift 2 ;;
    --dp) dp="$2"; shift 2 ;;
    --ep) ep="$2"; shift 2 ;;
    --seq-len) seq="$2"; shift 2 ;;
    --batch|--batch-size) batch="$2"; shift 2 ;;
    --steps|--iters) steps="$2"; shift 2 ;;
    --bmm-experts) bmm=1; shift ;;
    *) echo "unknown argument: $1" >&2; exit 2 ;;
  esac
done
if ! "${PYTHON:-python}" -c "import torchtitan.train" >/dev/null 2>&1; then
  echo "run_torchtitan.sh: torchtitan is not installed" >&2
  exit 3
fi
if ((bmm)); then
  export TORCHTITAN_USE_BMM_EXPERTS=1
  export PYTHONPATH="$HERE/..${PYTHONPATH:+:$PYTHONPATH}"
fi
exec torchrun --nnodes=1 --nproc-per-node="$gpus" --master-addr 127.0.0.1 -m torchtitan.train \
  --model.name qwen3 --model.flavor "$flavor" \
  --parallelism.pipeline_parallel_degree "$pp" --parallelism.data_parallel_replicate_degree "$dp" \
  --parallelism.expert_parallel_degree "$ep" --parallelism.pipeline_parallel_schedule 1F1B \
  --training.seq_len "$seq" --training.local_batch_size "$batch" --training.steps "$steps" \
  --training.dataset c4_test --metrics.log_freq 1
