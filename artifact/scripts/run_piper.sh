#!/usr/bin/env bash
# One experiment of the end-to-end evaluation on this framework.
#
#   artifact/scripts/run_piper.sh --model 1B --schedule 1f1b --pp 2 --dp 2 [--ep] [--zero-stage 0|1|2|3]
#       [--bucket-size MB] [--batch-size N] [--seq-len N] [--mbs N] [--warmup N] [--iters N]
#       [--metrics-out FILE] [--device cuda|cpu] [--dtype bf16|fp32]
#
# Builds the base schedule for the requested layout, runs it through examples/test_harness.py (one process per
# GPU on this box; there is no Ray cluster to join, so --address/--port/--temp-dir are accepted and ignored) and
# copies the run's results.csv to --metrics-out.
set -euo pipefail

HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(cd "$HERE/../.." && pwd)"
PY="${PYTHON:-python}"

model=1B; schedule=1f1b; pp=1; dp=1; ep=0; zero=1; bucket=""; batch=4; seq=512; mbs=1; warmup=3; iters=10
sleep_s=0; metrics=""; device=""; dtype=bf16; extra=()

while (($#)); do
  case "$1" in
    --model) model="$2"; shift 2 ;;
    --schedule) schedule="$2"; shift 2 ;;
    --pp) pp="$2"; shift 2 ;;
    --dp) dp="$2"; shift 2 ;;
    --ep) ep=1; shift ;;
    --zero-stage) zero="$2"; shift 2 ;;
    --bucket-size) bucket="$2"; shift 2 ;;
    --batch-size) batch="$2"; shift 2 ;;
    --seq-len) seq="$2"; shift 2 ;;
    --mbs) mbs="$2"; shift 2 ;;
    --warmup) warmup="$2"; shift 2 ;;
    --iters) iters="$2"; shift 2 ;;
    --iteration-sleep) sleep_s="$2"; shift 2 ;;
    --metrics-out) metrics="$2"; shift 2 ;;
    --device) device="$2"; shift 2 ;;
    --dtype) dtype="$2"; shift 2 ;;
    --address|--port|--temp-dir) shift 2 ;;                       # Ray cluster options of the reference
    --nsight|--use-inductor|--no-use-inductor|--pp-outer|--no-pp-outer) extra+=("$1"); shift ;;
    --gradient-accumulation|--no-gradient-accumulation|--ar-a2a-same-stream|--no-ar-a2a-same-stream) shift ;;
    --overlap-chunks|--no-overlap-chunks) shift ;;
    *) echo "unknown argument: $1" >&2; exit 2 ;;
  esac
done

# schedule name of the evaluation -> harness schedule and virtual stages per rank
case "$schedule" in
  1f1b) harness_schedule=1f1b; virtual=1 ;;
  interleaved1f1b|interleaved-1f1b|interleaved_1f1b) harness_schedule=interleaved_1f1b; virtual=2 ;;
  zerobubble|interleaved-zerobubble|interleavedzerobubble) harness_schedule=zerobubble; virtual=1 ;;
  dualpipe|dualpipev) harness_schedule=dualpipev; virtual=2 ;;
  *) echo "unknown schedule: $schedule" >&2; exit 2 ;;
esac

run_dir="$(mktemp -d "${TMPDIR:-/tmp}/piper_run.XXXXXX")"
base="$run_dir/base.json"
gen=("$PY" "$HERE/make_piper_base_schedule.py" --pp "$pp" --dp "$dp" --virtual-stages "$virtual"
     --zero "$zero" --out "$base")
((ep)) && gen+=(--ep)
[[ "$harness_schedule" == dualpipev ]] && gen+=(--v-placement)
[[ -n "$bucket" ]] && gen+=(--bucket-size "$bucket")
"${gen[@]}"

cmd=("$PY" "$ROOT/examples/test_harness.py" --test-file "$ROOT/examples/test_qwen.py" --base-schedule "$base"
     --schedule "$harness_schedule" --ranks "$pp" --mbs "$mbs" --out-root "$run_dir/out"
     --model "$model" --batch-size "$batch" --seq-len "$seq" --warmup "$warmup" --iters "$iters"
     --dtype "$dtype")
[[ "$sleep_s" != 0 ]] && cmd+=(--iteration-sleep "$sleep_s")
[[ -n "$device" ]] && cmd+=(--device "$device")
((${#extra[@]})) && cmd+=("${extra[@]}")
echo "[run_piper] ${cmd[*]}"
(cd "$ROOT" && "${cmd[@]}")

csv="$(find "$run_dir/out" -name results.csv | head -n 1)"
if [[ -n "$metrics" && -n "$csv" ]]; then
  mkdir -p "$(dirname "$metrics")"
  cp "$csv" "$metrics"
fi
echo "[run_piper] results: ${csv:-none}"
