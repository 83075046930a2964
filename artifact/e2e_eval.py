"""End-to-end evaluation driver: experiment matrix -> backend -> logs -> results.csv (+ bar charts).

``python artifact/e2e_eval.py --backend local --systems piper --sweeps local [--dry-run]``

Sweeps (the reference's paper experiments, ``artifact/e2e_eval.py:137-281``):

* ``scalability``  qwen 9B, pp in {4, 8} x dp in {1, 2, 4}, micro-batch 4, seq 512, 1F1B
* ``zero``         qwen 1B, pp8 x dp2, micro-batch in {16, 24, 32, 34, 36, 38, 40}, zero 1/2/3
* ``schedule``     qwen 9B, pp2 x dp2 x ep2, {1f1b, interleaved_1f1b, zerobubble, dualpipev}
* ``local``        small configurations that fit one 8-GPU box (or CPU ranks with ``--device cpu``)

Systems: ``piper`` (this framework, through ``examples/test_harness.py``) and the baseline runners of the
reference's artifact (``torchtitan``, ``megatron``, ``deepspeed``); a baseline that is not installed where the
command would run is recorded as skipped.

Backends (``artifact/e2e_eval.py:478-763`` of the reference):

* ``local``   runs every command as a subprocess on this machine, or inside ``docker run`` when ``--image`` is
              given (GPU selection through ``--cuda-visible-devices``);
* ``ssh``     (alias ``aws``) runs on a head node and workers reached over ssh (``SSH_KEY``, ``HEAD_PUBLIC_IP``,
              ``HEAD_PRIVATE_IP``, ``WORKER<i>_PRIVATE_IP``; workers are reached through the head node).  This
              framework needs one command on the head node (its launcher starts the ranks); the baselines get
              one command per node with ``NODE_RANK`` set.  Logs of all nodes are concatenated.

Every run leaves ``<out>/<run_id>/<system>/<sweep>_<name>.log``; ``parse_log`` turns a log (and, for ``piper``,
the harness's ``results.csv``) into mean/std iteration time, peak memory per rank and an out-of-memory flag.
``results.csv`` has one row per (system, experiment) with tokens/s = global batch x sequence length / mean
iteration time; ``<sweep>.svg`` bar charts are drawn without matplotlib.
"""
from __future__ import annotations

import argparse
import csv
import importlib.util
import itertools
import json
import math
import os
import re
import shlex
import subprocess
import sys
import tempfile
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Optional, Sequence

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "artifact" / "scripts"))

CONTAINER_ROOT = "/workspace/piper"


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


@dataclass
class Result:
    system: str
    sweep: str
    name: str
    model: str
    schedule: str
    pp: int
    dp: int
    ep: bool
    zero: int
    micro_batch: int
    num_microbatches: int
    seq_len: int
    gpus: int
    global_batch: int
    status: str = "dry-run"
    iter_time_mean_s: Optional[float] = None
    iter_time_std_s: Optional[float] = None
    tokens_per_s: Optional[float] = None
    peak_memory_gb: str = ""
    oom: bool = False
    command: str = ""


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


# ------------------------------------------------------------------------------------------------ commands
def piper_command(exp: Experiment, run_dir: Path, device: Optional[str], dtype: str) -> list[str]:
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


def baseline_command(system: str, exp: Experiment) -> Optional[list[str]]:
    """Command lines of the baseline runners; ``{nnode}``, ``{ngpu}``, ``{node_rank}`` and ``{master_addr}`` are
    filled in per node by the backend."""
    launch = ["torchrun", "--nnodes={nnode}", "--nproc-per-node={ngpu}", "--node-rank={node_rank}",
              "--master-addr={master_addr}", "--master-port=29500"]
    if system == "torchtitan":
        return launch + ["-m", "torchtitan.train", "--model.name", "qwen3", "--model.flavor", exp.model,
                         "--parallelism.pipeline_parallel_degree", str(exp.pp),
                         "--parallelism.data_parallel_replicate_degree", str(exp.dp),
                         "--training.seq_len", str(exp.seq_len),
                         "--training.local_batch_size", str(exp.micro_batch * exp.num_microbatches)]
    if system == "megatron":
        return launch + ["pretrain_gpt.py", "--pipeline-model-parallel-size", str(exp.pp), "--micro-batch-size",
                         str(exp.micro_batch), "--global-batch-size", str(exp.global_batch), "--seq-length",
                         str(exp.seq_len), "--tensor-model-parallel-size", "1"]
    if system == "deepspeed":
        return launch + [str(ROOT / "artifact" / "run_deepspeed.py"), "--pp", str(exp.pp), "--zero", str(exp.zero),
                         "--micro-batch", str(exp.micro_batch), "--seq-len", str(exp.seq_len)]
    return None


def render(command: Sequence[str], *, nnode: int, ngpu: int, node_rank: int, master_addr: str) -> list[str]:
    vals = {"nnode": nnode, "ngpu": ngpu, "node_rank": node_rank, "master_addr": master_addr}
    return [part.format(**vals) if "{" in part else part for part in command]


def system_available(system: str) -> bool:
    if system == "piper":
        return True
    return importlib.util.find_spec(system) is not None


# ------------------------------------------------------------------------------------------------ backends
class Backend:
    """Where and how a command runs.  ``layout`` maps an experiment to (nodes, GPUs per node)."""
    name = "backend"

    def layout(self, exp: Experiment) -> tuple[int, int]:
        return 1, exp.gpus

    def run(self, system: str, exp: Experiment, command: Sequence[str], log_path: Path, timeout: float) -> int:
        raise NotImplementedError

    def dry_run_lines(self, system: str, exp: Experiment, command: Sequence[str]) -> list[str]:
        raise NotImplementedError


class LocalBackend(Backend):
    """Subprocesses on this machine; with ``image`` the command runs inside ``docker run --gpus``."""
    name = "local"

    def __init__(self, image: Optional[str] = None, cuda_visible_devices: Optional[str] = None,
                 docker_args: Sequence[str] = ()) -> None:
        self.image = image
        self.cuda_visible_devices = cuda_visible_devices
        self.docker_args = list(docker_args)

    def _wrap(self, rendered: list[str], out_dir: Optional[Path] = None) -> list[str]:
        if not self.image:
            return rendered
        gpus = "all" if self.cuda_visible_devices is None else f'"device={self.cuda_visible_devices}"'
        cmd = ["docker", "run", "--rm", "--gpus", gpus, "--network", "host", "--ipc", "host", "--shm-size", "32g",
               "-v", f"{ROOT}:{CONTAINER_ROOT}", "-w", CONTAINER_ROOT]
        if out_dir is not None:
            cmd += ["-v", f"{out_dir}:{out_dir}"]
        cmd += [*self.docker_args, self.image, "bash", "-lc",
                shlex.join(rendered).replace(str(ROOT), CONTAINER_ROOT)]
        return cmd

    def _env(self) -> dict:
        env = dict(os.environ)
        if self.cuda_visible_devices is not None and not self.image:
            env["CUDA_VISIBLE_DEVICES"] = self.cuda_visible_devices
        return env

    def run(self, system, exp, command, log_path, timeout):
        nnode, ngpu = self.layout(exp)
        rendered = render(command, nnode=nnode, ngpu=ngpu, node_rank=0, master_addr="127.0.0.1")
        log_path.parent.mkdir(parents=True, exist_ok=True)
        with log_path.open("w", encoding="utf-8") as f:
            try:
                return subprocess.run(self._wrap(rendered, log_path.parent.parent), stdout=f, stderr=subprocess.STDOUT,
                                      timeout=timeout, cwd=str(ROOT), env=self._env()).returncode
            except subprocess.TimeoutExpired:
                f.write(f"\n[e2e_eval] timed out after {timeout}s\n")
                return -1

    def dry_run_lines(self, system, exp, command):
        nnode, ngpu = self.layout(exp)
        return [shlex.join(self._wrap(render(command, nnode=nnode, ngpu=ngpu, node_rank=0, master_addr="127.0.0.1")))]


class SshBackend(Backend):
    """A head node and workers reached over ssh; commands run inside a named container on each node."""
    name = "ssh"

    def __init__(self, container: str = "piper-e2e", gpus_per_node: int = 8, dry: bool = False) -> None:
        def need(var: str) -> str:
            v = os.environ.get(var)
            if not v and not dry:
                raise SystemExit(f"the ssh backend needs the environment variable {var}")
            return v or f"<{var}>"

        self.key, self.head_public, self.head_private = need("SSH_KEY"), need("HEAD_PUBLIC_IP"), need("HEAD_PRIVATE_IP")
        self.workers = []
        i = 1
        while os.environ.get(f"WORKER{i}_PRIVATE_IP"):
            self.workers.append(os.environ[f"WORKER{i}_PRIVATE_IP"])
            i += 1
        self.container, self.gpus_per_node = container, gpus_per_node

    def layout(self, exp):
        nnode = max(1, math.ceil(exp.gpus / self.gpus_per_node))
        return nnode, min(exp.gpus, self.gpus_per_node)

    def _ssh(self, target: str, remote: str, through_head: bool) -> list[str]:
        cmd = ["ssh", "-i", self.key, "-o", "StrictHostKeyChecking=no"]
        if through_head:
            cmd += ["-o", f"ProxyCommand=ssh -i {self.key} -o StrictHostKeyChecking=no -W %h:%p ubuntu@{self.head_public}"]
        return cmd + [f"ubuntu@{target}", remote]

    def _nodes(self, nnode: int) -> list[tuple[str, str, bool]]:
        if nnode - 1 > len(self.workers):
            raise RuntimeError(f"{nnode} nodes requested but only {len(self.workers)} WORKER<i>_PRIVATE_IP values are set")
        return [("head", self.head_public, False)] + [(f"worker{i + 1}", ip, True)
                                                      for i, ip in enumerate(self.workers[:nnode - 1])]

    def _remote(self, rendered: list[str], node_rank: int) -> str:
        inner = shlex.join(rendered).replace(str(ROOT), CONTAINER_ROOT)
        return shlex.join(["docker", "exec", "-e", f"NODE_RANK={node_rank}", self.container, "bash", "-lc", inner])

    def _per_node(self, system: str, exp: Experiment, command: Sequence[str]) -> list[tuple[str, list[str]]]:
        nnode, ngpu = self.layout(exp)
        nodes = self._nodes(nnode)
        if system == "piper":
            nodes = nodes[:1]          # this framework's launcher starts every rank from the head node
        out = []
        for rank, (label, target, via_head) in enumerate(nodes):
            rendered = render(command, nnode=nnode, ngpu=ngpu, node_rank=rank, master_addr=self.head_private)
            out.append((label, self._ssh(target, self._remote(rendered, rank), via_head)))
        return out

    def run(self, system, exp, command, log_path, timeout):
        log_path.parent.mkdir(parents=True, exist_ok=True)
        with tempfile.TemporaryDirectory(prefix="piper-e2e-") as tmp:
            procs = []
            for label, cmd in self._per_node(system, exp, command):
                node_log = Path(tmp) / f"{label}.log"
                procs.append((label, node_log, subprocess.Popen(cmd, stdout=node_log.open("w"), stderr=subprocess.STDOUT)))
            codes = []
            deadline = time.monotonic() + timeout
            for _label, _log, p in procs:
                try:
                    codes.append(p.wait(max(1.0, deadline - time.monotonic())))
                except subprocess.TimeoutExpired:
                    p.kill()
                    codes.append(-1)
            with log_path.open("w", encoding="utf-8") as combined:
                for label, node_log, _p in procs:
                    combined.write(f"===== {label} =====\n{node_log.read_text(errors='replace')}\n")
        return next((c for c in codes if c != 0), 0)

    def dry_run_lines(self, system, exp, command):
        return [f"{label}: {shlex.join(cmd)}" for label, cmd in self._per_node(system, exp, command)]


# ------------------------------------------------------------------------------------------------- parsing
ANSI = re.compile(r"\x1b\[[0-9;]*[A-Za-z]")
OOM = re.compile(r"out of memory|OutOfMemoryError|CUDA_ERROR_OUT_OF_MEMORY", re.I)
# TorchTitan: "step: 10  loss: 7.1  memory: 31.20GiB(39.0%)  tps: 5,120 ..." (rank-prefixed lines carry "[rankN]")
TT_STEP = re.compile(r"(?:\[rank(\d+)\])?.*?step:\s*(\d+).*?memory:\s*([0-9.]+)\s*GiB.*?tps:\s*([0-9,\.]+)", re.I)
# Megatron-LM: "elapsed time per iteration (ms): 1234.5" and "[Rank 3] (after N iterations) memory (MB) | ... max allocated: X"
MG_ITER = re.compile(r"elapsed time per iteration \(ms\):\s*([0-9.]+)")
MG_MEM = re.compile(r"\[Rank (\d+)\].*?max allocated:\s*([0-9.]+)")
# artifact/run_deepspeed.py: "[step 7] loss=... time=0.412s", "peak memory rank 0: 12.3 GB"
DS_STEP = re.compile(r"\[step \d+\].*?time=([0-9.]+)s")
DS_MEM = re.compile(r"peak memory rank (\d+):\s*([0-9.]+)\s*GB", re.I)


def _mean_std(values: Sequence[float]) -> tuple[Optional[float], Optional[float]]:
    if not values:
        return None, None
    m = sum(values) / len(values)
    return m, math.sqrt(sum((v - m) ** 2 for v in values) / len(values))


def parse_log(system: str, log_path: Path, metrics_csv: Optional[Path] = None, tokens_per_iter: int = 0) -> dict:
    """Mean/std iteration time (s), peak memory per rank and the out-of-memory flag of one run."""
    text = ANSI.sub("", log_path.read_text(errors="replace").replace("\0", "")) if log_path.is_file() else ""
    out = {"iter_time_mean_s": None, "iter_time_std_s": None, "peak_memory_gb": "", "oom": OOM.search(text) is not None}
    if system == "piper":
        if metrics_csv is not None and metrics_csv.is_file():
            rows = list(csv.DictReader(metrics_csv.open()))
            means, stds, peaks = [], [], []
            for r in rows:
                try:
                    means.append(float(r["iter_time_mean_s"]))
                    stds.append(float(r.get("iter_time_std_s") or 0.0))
                except (KeyError, ValueError):
                    continue
                peaks += [f"{k[len('peak_memory_pp'):-len('_gb')]}:{float(v):.2f}" for k, v in r.items()
                          if k.startswith("peak_memory_pp") and v]
            if means:
                # replicas step together: the slowest replica's mean is the job's iteration time
                out.update(iter_time_mean_s=max(means), iter_time_std_s=max(stds), peak_memory_gb=";".join(sorted(set(peaks))))
        return out
    if system == "torchtitan":
        per_rank: dict[int, list] = {}
        for m in TT_STEP.finditer(text):
            rank = int(m.group(1) or 0)
            per_rank.setdefault(rank, []).append((float(m.group(3)), float(m.group(4).replace(",", ""))))
        if per_rank and tokens_per_iter:
            tps = [t for _mem, t in per_rank[min(per_rank)]][-5:]
            ranks = max(1, len(per_rank))
            times = [tokens_per_iter / (t * ranks) for t in tps if t > 0]      # tps is per rank
            out["iter_time_mean_s"], out["iter_time_std_s"] = _mean_std(times)
        out["peak_memory_gb"] = "/".join(f"{max(mem for mem, _t in v):.2f}" for _r, v in sorted(per_rank.items()))
        return out
    if system == "megatron":
        out["iter_time_mean_s"], out["iter_time_std_s"] = _mean_std([float(v) / 1e3 for v in MG_ITER.findall(text)][-5:])
        peak = {int(r): float(v) / 1024.0 for r, v in MG_MEM.findall(text)}
        out["peak_memory_gb"] = "/".join(f"{peak[r]:.2f}" for r in sorted(peak))
        return out
    if system == "deepspeed":
        out["iter_time_mean_s"], out["iter_time_std_s"] = _mean_std([float(v) for v in DS_STEP.findall(text)][-5:])
        peak = {int(r): float(v) for r, v in DS_MEM.findall(text)}
        out["peak_memory_gb"] = "/".join(f"{peak[r]:.2f}" for r in sorted(peak))
    return out


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


def write_results(run_dir: Path, rows: list[Result]) -> Path:
    out_csv = run_dir / "results.csv"
    with out_csv.open("w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(Result.__annotations__.keys()))
        w.writeheader()
        for r in rows:
            w.writerow(asdict(r))
    for sweep in sorted({r.sweep for r in rows}):
        sel = [r for r in rows if r.sweep == sweep and r.tokens_per_s]
        if sel:
            bar_chart_svg(f"{sweep}: tokens/s", [f"{r.system}:{r.name}" for r in sel], [r.tokens_per_s for r in sel],
                          run_dir / f"{sweep}.svg")
    return out_csv


# --------------------------------------------------------------------------------------------------- driver
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--backend", choices=("local", "ssh", "aws"), default="local")
    ap.add_argument("--systems", default="piper")
    ap.add_argument("--sweeps", default="local")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--device", default=None)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--image", default=None, help="local backend: run inside `docker run` with this image")
    ap.add_argument("--cuda-visible-devices", default=None)
    ap.add_argument("--container", default="piper-e2e", help="ssh backend: container name on every node")
    ap.add_argument("--gpus-per-node", type=int, default=8)
    ap.add_argument("--out", default=str(ROOT / "artifact" / "out" / "e2e-eval"))
    ap.add_argument("--timeout", type=float, default=3600)
    a = ap.parse_args(argv)
    run_dir = Path(a.out) / time.strftime("%Y%m%d_%H%M%S")
    run_dir.mkdir(parents=True, exist_ok=True)
    backend: Backend = (LocalBackend(a.image, a.cuda_visible_devices) if a.backend == "local"
                        else SshBackend(a.container, a.gpus_per_node, dry=a.dry_run))
    systems = [s for s in a.systems.split(",") if s]
    rows: list[Result] = []
    for exp in build_matrix([s for s in a.sweeps.split(",") if s]):
        for system in systems:
            cmd = piper_command(exp, run_dir, a.device, a.dtype) if system == "piper" else baseline_command(system, exp)
            if cmd is None:
                continue
            row = Result(system=system, sweep=exp.sweep, name=exp.name, model=exp.model, schedule=exp.schedule,
                         pp=exp.pp, dp=exp.dp, ep=exp.ep, zero=exp.zero, micro_batch=exp.micro_batch,
                         num_microbatches=exp.num_microbatches, seq_len=exp.seq_len, gpus=exp.gpus,
                         global_batch=exp.global_batch)
            lines = backend.dry_run_lines(system, exp, cmd)
            row.command = " && ".join(lines)
            if a.dry_run:
                print("\n".join(lines))
            elif a.backend == "local" and not a.image and not system_available(system):
                row.status = "skipped: not installed"
            else:
                log = run_dir / system / f"{exp.sweep}_{exp.name}.log"
                rc = backend.run(system, exp, cmd, log, a.timeout)
                metrics = None
                if system == "piper":
                    found = sorted((run_dir / "piper" / f"{exp.sweep}_{exp.name}").glob("*/results.csv"))
                    metrics = found[-1] if found else None
                parsed = parse_log(system, log, metrics, tokens_per_iter=exp.global_batch * exp.seq_len)
                row.status = "ok" if rc == 0 else ("oom" if parsed["oom"] else f"failed rc={rc}")
                row.iter_time_mean_s, row.iter_time_std_s = parsed["iter_time_mean_s"], parsed["iter_time_std_s"]
                row.peak_memory_gb, row.oom = parsed["peak_memory_gb"], parsed["oom"]
                if row.iter_time_mean_s:
                    row.tokens_per_s = exp.global_batch * exp.seq_len / row.iter_time_mean_s
            rows.append(row)
    print(f"results written to {write_results(run_dir, rows)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
