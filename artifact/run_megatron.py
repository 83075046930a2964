"""Baseline runner: Megatron-LM on the evaluation's MoE shapes with mock data.

Builds the ``pretrain_gpt.py`` command for one experiment (model shape, tp/pp/dp/ep/cp degrees, micro and global
batch, sequence length, iterations), launches it with ``torchrun`` and reports tokens/s parsed from Megatron's
own "elapsed time per iteration (ms)" log lines.  Megatron-LM is not part of this repository: point
``MEGATRON_HOME`` at a checkout (the directory holding ``pretrain_gpt.py``).  ``--dry-run`` prints the command
without needing one.  Counterpart of the reference artifact's ``artifact/run_megatron.py:100-349``.
"""
from __future__ import annotations

import argparse
import os
import re
import shlex
import subprocess
import sys
from pathlib import Path

# name -> (layers, hidden, q heads, kv heads, head_dim, experts, top_k, expert ffn, vocab)
MODEL_SHAPES = {
    "qwen3_1b": (16, 1024, 16, 4, 128, 32, 4, 512, 151936),
    "qwen3_9b": (32, 2048, 32, 4, 128, 64, 8, 768, 151936),
    "qwen3_30b_a3b": (48, 2048, 32, 4, 128, 128, 8, 768, 151936),
}

_ITER_MS = re.compile(r"elapsed time per iteration \(ms\):\s*([0-9.]+)")


def build_command(a: argparse.Namespace, megatron_home: str) -> list[str]:
    layers, hidden, heads, kv, hd, experts, top_k, ffn, vocab = MODEL_SHAPES[a.model]
    world = a.nnodes * a.nproc_per_node
    need = a.tp * a.pp * a.dp * a.cp
    if need != world:
        raise SystemExit(f"tp*pp*dp*cp = {need} does not match nnodes*nproc-per-node = {world}")
    launch = ["torchrun", f"--nnodes={a.nnodes}", f"--nproc-per-node={a.nproc_per_node}",
              f"--master-addr={a.master_addr or '127.0.0.1'}", f"--master-port={a.master_port}"]
    model = ["--num-layers", str(layers), "--hidden-size", str(hidden), "--num-attention-heads", str(heads),
             "--group-query-attention", "--num-query-groups", str(kv), "--kv-channels", str(hd),
             "--ffn-hidden-size", str(ffn), "--moe-ffn-hidden-size", str(ffn), "--num-experts", str(experts),
             "--moe-router-topk", str(top_k), "--moe-grouped-gemm", "--moe-token-dispatcher-type", "alltoall",
             "--swiglu", "--normalization", "RMSNorm", "--qk-layernorm", "--position-embedding-type", "rope",
             "--rotary-base", "1000000", "--untie-embeddings-and-output-weights", "--disable-bias-linear",
             "--vocab-size", str(vocab), "--max-position-embeddings", str(a.seq_length)]
    par = ["--tensor-model-parallel-size", str(a.tp), "--pipeline-model-parallel-size", str(a.pp),
           "--context-parallel-size", str(a.cp), "--expert-model-parallel-size", str(a.ep)]
    if a.sp:
        par.append("--sequence-parallel")
    if a.use_tp_pp_dp_mapping:
        par.append("--use-tp-pp-dp-mapping")
    train = ["--micro-batch-size", str(a.micro_bs), "--global-batch-size", str(a.global_bs), "--seq-length",
             str(a.seq_length), "--train-iters", str(a.train_iters), "--bf16", "--lr", "1e-4", "--min-lr", "1e-5",
             "--lr-decay-style", "constant", "--mock-data", "--tokenizer-type", "NullTokenizer", "--log-interval", "1",
             "--eval-iters", "0", "--no-save-optim", "--no-save-rng", "--tensorboard-dir", a.tensorboard_dir,
             "--rerun-mode", a.rerun_mode, "--use-distributed-optimizer", "--overlap-grad-reduce",
             "--use-mcore-models", "--transformer-impl", "transformer_engine"]
    cmd = launch + [str(Path(megatron_home) / "pretrain_gpt.py")] + model + par + train
    if a.nsight:
        cmd = ["nsys", "profile", "-o", "megatron_%p", "--trace=cuda,nvtx"] + cmd
    return cmd


def tokens_per_second(log_text: str, global_bs: int, seq_length: int, skip: int = 3) -> float | None:
    """Mean tokens/s over the logged iterations after ``skip`` warm-up iterations."""
    ms = [float(m) for m in _ITER_MS.findall(log_text)][skip:]
    if not ms:
        return None
    return global_bs * seq_length / (sum(ms) / len(ms) / 1e3)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--model", choices=tuple(MODEL_SHAPES), default="qwen3_30b_a3b")
    p.add_argument("--tensorboard-dir", default="tensorboard/moe_mock")
    p.add_argument("--micro-bs", type=int, default=16)
    p.add_argument("--global-bs", type=int, default=64)
    p.add_argument("--train-iters", type=int, default=8)
    for name in ("tp", "pp", "dp", "cp", "ep"):
        p.add_argument(f"--{name}", type=int, default=1)
    p.add_argument("--seq-length", type=int, default=512)
    p.add_argument("--sp", action="store_true")
    p.add_argument("--use-tp-pp-dp-mapping", action="store_true")
    p.add_argument("--nnodes", type=int, required=True)
    p.add_argument("--nproc-per-node", type=int, required=True)
    p.add_argument("--master-addr", default=None)
    p.add_argument("--master-port", default="6000")
    p.add_argument("--nsight", action="store_true")
    p.add_argument("--rerun-mode", choices=("disabled", "validate_results", "report_stats"), default="disabled")
    p.add_argument("--dry-run", action="store_true")
    a = p.parse_args(argv)

    home = os.environ.get("MEGATRON_HOME", "")
    cmd = build_command(a, home or "$MEGATRON_HOME")
    if a.dry_run:
        print(shlex.join(cmd))
        return 0
    if not home or not (Path(home) / "pretrain_gpt.py").exists():
        print("run_megatron: Megatron-LM not found (set MEGATRON_HOME to a checkout holding pretrain_gpt.py)",
              file=sys.stderr)
        return 3
    env = dict(os.environ, CUDA_DEVICE_MAX_CONNECTIONS="1", PYTHONPATH=home + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    sys.stdout.write(proc.stdout)
    tps = tokens_per_second(proc.stdout, a.global_bs, a.seq_length)
    if tps is not None:
        print(f"throughput tokens/s: {tps:.1f}")
    return proc.returncode


if __name__ == "__main__":
    sys.exit(main())
