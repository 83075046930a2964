"""End-to-end evaluation driver: experiment matrix -> commands -> logs -> results.csv (+ bar charts).

``python artifact/e2e_eval.py --backend local --systems piper --sweeps local [--dry-run]``

Sweeps (definitions of the reference's paper experiments, ``artifact/e2e_eval.py:149-186``):

* ``scalability``  qwen 9B, pp in {4, 8} x dp in {1, 2, 4}, micro-batch 4, seq 512, 1F1B
* ``zero``         qwen 1B, pp8 x dp2, micro-batch in {16, 24, 32, 34, 36, 38, 40}, zero 1/2/3
* ``schedule``     qwen 9B, pp2 x dp2 x ep2, {1f1b, interleaved_1f1b, zerobubble, dualpipev}
* ``local``        small configurations that fit one 8-GPU box (or CPU ranks with ``--device cpu``)

Systems: ``piper`` (this framework, through ``examples/test_harness.py``) and the baseline runners of the
reference's artifact (``torchtitan``, ``megatron``, ``deepspeed``), for which only the command lines are built:
those packages are not part of this repository and are skipped unless importable.  Backends: ``local`` runs
the commands as subprocesses on this machine; ``ssh`` prefixes them with ``ssh <host>`` for a head node given by
``HEAD_PUBLIC_IP`` / ``SSH_KEY`` (dry-run prints them).  Results: ``artifact/out/e2e-eval/<run_id>/results.csv``,
one row per (system, experiment), tokens/s = global_batch * seq_len / mean iteration time; ``<sweep>.svg`` bar
charts are drawn without matplotlib.
"""
from __future__ import annotations

import argparse
import csv
import importlib.util
import itertools
import json
import os
import re
import subprocess
import sys
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "artifact" / "scripts"))


@dataclass
class Experiment:
    sweep: str
    name: str
    model: str
    family: str = "qwen"
    pp: int = 1
    dp: int = 1
    ep: bool = False
    zero: int = 0
    schedule: str = "1f1b"
    micro_batch: int = 1
    num_microbatches: int = 4
    seq_len: int = 512
    virtual_stages: int = 1
    extra: dict = field(default_factory=dict)

    @property
    def gpus(self) -> int:
        return self.pp * self.dp

    @property
    def global_batch(self) -> int:
        return self.micro_batch * self.num_microbatches * self.dp


def build_matrix(sweeps: list[str]) -> list[Experiment]:
    out: list[Experiment] = []
    if "scalability" in sweeps:
        for pp, dp in itertools.product((4, 8), (1, 2, 4)):
            out.append(Experiment("scalability", f"pp{pp}_dp{dp}", "9B", pp=pp, dp=dp, micro_batch=4,
                                  num_microbatches=2 * pp, seq_len=512))
    if "zero" in sweeps:
        for mb, z in itertools.product((16, 24, 32, 34, 36, 38, 40), (1, 2, 3)):
            out.append(Experiment("zero", f"mb{mb}_zero{z}", "1B", pp=8, dp=2, zero=z, micro_batch=mb,
                                  num_microbatches=16, seq_len=512))
    if "schedule" in sweeps:
        for sched in ("1f1b", "interleaved_1f1b", "zerobubble", "dualpipev"):
            v = 2 if sched in ("interleaved_1f1b", "dualpipev") else 1
            out.append(Experiment("schedule", sched, "9B", pp=2, dp=2, ep=True, schedule=sched, micro_batch=4,
                                  num_microbatches=8, seq_len=512, virtual_stages=v))
    if "local" in sweeps:
        out.append(Experiment("local", "llama_debug_dp2", "debug", family="llama", pp=1, dp=2, micro_batch=1,
                              num_microbatches=2, seq_len=128))
        out.append(Experiment("local", "qwen_9M_pp2_dp2_ep2", "9M", pp=2, dp=2, ep=True, micro_batch=1,
                              num_microbatches=4, seq_len=128))
        out.append(Experiment("local", "qwen_9M_dualpipev", "9M", pp=2, dp=2, ep=True, schedule="dualpipev",
                              micro_batch=1, num_microbatches=4, seq_len=128, virtual_stages=2))
    return out


def piper_command(exp: Experiment, run_dir: Path, device: str | None, dtype: str) -> list[str]:
    from make_piper_base_schedule import make_schedule

    sched = make_schedule(exp.pp, exp.dp, exp.zero, exp.ep, exp.virtual_stages, v_placement=exp.schedule == "dualpipev")
    base = run_dir / "schedules" / f"{exp.sweep}_{exp.name}.json"
    base.parent.mkdir(parents=True, exist_ok=True)
    base.write_text(json.dumps(sched, indent=2))
    driver = "test_llama.py" if exp.family == "llama" else "test_qwen.py"
    cmd = [sys.executable, str(ROOT / "examples" / "test_harness.py"), "--test-file", str(ROOT / "examples" / driver),
           "--base-schedule", str(base), "--schedule", exp.schedule, "--ranks", str(exp.pp), "--mbs",
           str(exp.num_microbatches), "--out-root", str(run_dir / "piper" / f"{exp.sweep}_{exp.name}"),
           "--model", exp.model, "--batch-size", str(exp.micro_batch), "--seq-len", str(exp.seq_len),
           "--warmup", "3", "--iters", "3", "--dtype", dtype]
    if device:
        cmd += ["--device", device]
    return cmd


def baseline_command(system: str, exp: Experiment) -> list[str] | None:
    """Command lines of the reference artifact's baseline runners (not shipped here; used when installed)."""
    if system == "torchtitan":
        return ["torchrun", f"--nproc-per-node={exp.gpus}", "-m", "torchtitan.train", "--model.name", "qwen3",
                "--model.flavor", exp.model, "--parallelism.pipeline_parallel_degree", str(exp.pp),
                "--parallelism.data_parallel_replicate_degree", str(exp.dp), "--training.seq_len", str(exp.seq_len),
                "--training.local_batch_size", str(exp.micro_batch * exp.num_microbatches)]
    if system == "megatron":
        return ["torchrun", f"--nproc-per-node={exp.gpus}", "pretrain_gpt.py", "--pipeline-model-parallel-size",
                str(exp.pp), "--micro-batch-size", str(exp.micro_batch), "--global-batch-size", str(exp.global_batch),
                "--seq-length", str(exp.seq_len), "--tensor-model-parallel-size", "1"]
    if system == "deepspeed":
        return ["deepspeed", f"--num_gpus={exp.gpus}", "run_deepspeed.py", "--pp", str(exp.pp), "--zero", str(exp.zero),
                "--micro-batch", str(exp.micro_batch), "--seq-len", str(exp.seq_len)]
    return None


def system_available(system: str) -> bool:
    if system == "piper":
        return True
    return importlib.util.find_spec({"torchtitan": "torchtitan", "megatron": "megatron", "deepspeed": "deepspeed"}[system]) is not None


_TOK = re.compile(r"throughput[^0-9]*([0-9.]+)|tokens?/s[^0-9]*([0-9.]+)", re.I)


def parse_piper_results(out_root: Path) -> dict | None:
    files = sorted(out_root.glob("*/results.csv"))
    if not files:
        return None
    rows = list(csv.DictReader(files[-1].open()))
    if not rows:
        return None
    mean_iter = max(float(r["iter_time_mean_s"]) for r in rows)
    tokens = sum(int(r["batch_size"]) * int(r["num_microbatches"]) * int(r["seq_len"]) for r in rows)
    peak = max((float(v) for r in rows for k, v in r.items() if k.startswith("peak_memory") and v), default=0.0)
    return {"iter_time_mean_s": mean_iter, "tokens_per_s": tokens / mean_iter, "peak_memory_gb": peak}


def parse_log_throughput(text: str) -> float | None:
    vals = [float(a or b) for a, b in _TOK.findall(text)]
    return vals[-1] if vals else None


def bar_chart_svg(title: str, labels: list[str], values: list[float], path: Path) -> None:
    w, h, pad = 90 * max(len(labels), 1) + 80, 320, 40
    top = max(values + [1e-9])
    bars = []
    for i, (l, v) in enumerate(zip(labels, values)):
        bh = (h - 2 * pad) * v / top
        x = pad + 20 + i * 90
        bars.append(f'<rect x="{x}" y="{h - pad - bh:.1f}" width="60" height="{bh:.1f}" fill="#4c78a8"/>'
                    f'<text x="{x + 30}" y="{h - pad + 14}" font-size="9" text-anchor="middle">{l}</text>'
                    f'<text x="{x + 30}" y="{h - pad - bh - 4:.1f}" font-size="9" text-anchor="middle">{v:.0f}</text>')
    path.write_text(f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}"><text x="{w / 2}" y="16" '
                    f'text-anchor="middle" font-size="12">{title}</text>{"".join(bars)}</svg>')


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--backend", choices=("local", "ssh", "aws"), default="local")
    ap.add_argument("--systems", default="piper")
    ap.add_argument("--sweeps", default="local")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--device", default=None)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--out", default=str(ROOT / "artifact" / "out" / "e2e-eval"))
    ap.add_argument("--timeout", type=float, default=3600)
    a = ap.parse_args(argv)
    run_dir = Path(a.out) / time.strftime("%Y%m%d_%H%M%S")
    run_dir.mkdir(parents=True, exist_ok=True)
    systems = [s for s in a.systems.split(",") if s]
    rows = []
    for exp in build_matrix([s for s in a.sweeps.split(",") if s]):
        for system in systems:
            cmd = piper_command(exp, run_dir, a.device, a.dtype) if system == "piper" else baseline_command(system, exp)
            if cmd is None:
                continue
            if a.backend in ("ssh", "aws"):
                host = os.environ.get("HEAD_PUBLIC_IP", "<head-node>")
                key = os.environ.get("SSH_KEY", "<key.pem>")
                cmd = ["ssh", "-i", key, f"ubuntu@{host}", " ".join(cmd)]
            row = {"system": system, **{k: v for k, v in asdict(exp).items() if k != "extra"}, "gpus": exp.gpus,
                   "global_batch": exp.global_batch, "status": "dry-run", "tokens_per_s": "", "iter_time_mean_s": "",
                   "peak_memory_gb": "", "command": " ".join(cmd)}
            if a.dry_run:
                print(row["command"])
            elif not system_available(system):
                row["status"] = "skipped: not installed"
            else:
                log = run_dir / system / f"{exp.sweep}_{exp.name}.log"
                log.parent.mkdir(parents=True, exist_ok=True)
                with log.open("w") as f:
                    try:
                        rc = subprocess.run(cmd, stdout=f, stderr=subprocess.STDOUT, timeout=a.timeout, cwd=str(ROOT)).returncode
                    except subprocess.TimeoutExpired:
                        rc = -1
                row["status"] = "ok" if rc == 0 else f"failed rc={rc}"
                if rc == 0 and system == "piper":
                    res = parse_piper_results(run_dir / "piper" / f"{exp.sweep}_{exp.name}")
                    if res:
                        row.update(res)
                elif rc == 0:
                    tp = parse_log_throughput(log.read_text())
                    if tp:
                        row["tokens_per_s"] = tp
            rows.append(row)
    out_csv = run_dir / "results.csv"
    with out_csv.open("w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(rows[0].keys()) if rows else ["system"])
        w.writeheader()
        w.writerows(rows)
    for sweep in sorted({r["sweep"] for r in rows}):
        sel = [r for r in rows if r["sweep"] == sweep and r["tokens_per_s"] not in ("", None)]
        if sel:
            bar_chart_svg(f"{sweep}: tokens/s", [f'{r["system"]}:{r["name"]}' for r in sel],
                          [float(r["tokens_per_s"]) for r in sel], run_dir / f"{sweep}.svg")
    print(f"results written to {out_csv}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
