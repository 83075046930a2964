"""Run the Qwen example configurations through the harness, one subprocess each, and report PASSED/FAILED.

Seven configurations as in the reference's batch runner (``examples/run_qwen_examples.py``): four schedules on
the PP2 x DP2 x EP2 base, the bucketed and ZeRO variants, interleaved placement and DualPipeV on the V placement.
``--device cpu --dtype fp32`` runs them on CPU ranks with gloo.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
BASE = HERE / "base-schedules"

EXAMPLES = [
    ("1f1b", "pp2_dp2_ep2.json", "1f1b", 2, 4),
    ("zerobubble", "pp2_dp2_ep2.json", "zerobubble", 2, 4),
    ("bucket100", "pp2_dp2_ep2_bucket100.json", "1f1b", 2, 4),
    ("zero2", "pp2_dp2_ep2_zero2.json", "1f1b", 2, 4),
    ("zero3", "pp2_dp2_ep2_zero3.json", "1f1b", 2, 4),
    ("interleaved", "pp4_dp2_ep2_interleaved.json", "interleaved_1f1b", 2, 4),
    ("dualpipev", "pp4_dp2_ep2_v_placement.json", "dualpipev", 2, 4),
]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", help="comma-separated example names")
    ap.add_argument("--model", default="9M")
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--device", default=None)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--timeout", type=float, default=1800)
    args = ap.parse_args()
    py = os.environ.get("PYTHON", sys.executable)
    only = {s for s in args.only.split(",") if s}
    results = []
    for name, base, sched, ranks, mbs in EXAMPLES:
        if only and name not in only:
            continue
        cmd = [py, str(HERE / "test_harness.py"), "--test-file", str(HERE / "test_qwen.py"), "--base-schedule",
               str(BASE / base), "--schedule", sched, "--ranks", str(ranks), "--mbs", str(mbs), "--model", args.model,
               "--seq-len", str(args.seq_len), "--batch-size", str(args.batch_size), "--warmup", "1", "--iters", "2",
               "--dtype", args.dtype]
        if args.device:
            cmd += ["--device", args.device]
        print("RUN", name, " ".join(cmd), flush=True)
        try:
            rc = subprocess.run(cmd, timeout=args.timeout).returncode
        except subprocess.TimeoutExpired:
            rc = -1
        results.append((name, rc))
        print(("PASSED" if rc == 0 else "FAILED"), name, flush=True)
    print("\n".join(f"{'PASSED' if rc == 0 else 'FAILED'} {n}" for n, rc in results))
    return 0 if all(rc == 0 for _, rc in results) else 1


if __name__ == "__main__":
    sys.exit(main())
