"""Shared body of the example drivers: set up, warm up, time, collect metrics.

A driver module exposes ``parse_args(argv)`` and ``main(args, pg) -> metrics dict`` (the contract of the
reference's ``examples/test_qwen.py`` / ``test_llama.py``); ``main`` runs in every rank of the job.  The
metrics keys are the reference's: ``dp_rank, model, schedule, schedule_directives_file, pp, dp, batch_size,
num_microbatches, seq_len, iter_times_s, peak_memory_by_rank``.  Iterations are timed on the device with
CUDA events when a GPU is used (the reference times a Ray round trip on the host).
"""
from __future__ import annotations

import argparse
import os
import time

import torch

from piper_b200 import piper_exec_dag, piper_setup
from piper_b200.compiler.schedule import load_schedule_directives
from piper_b200.state import LOG_LEVEL, create_logger, piper_metadata

logger = create_logger("piper_example", LOG_LEVEL)


def derive_num_stages(schedule_directives_file: str) -> int:
    n = sum(1 for d in load_schedule_directives(schedule_directives_file) if isinstance(d, dict) and d.get("op") == "place")
    if n <= 0:
        raise ValueError(f"schedule directives file must contain at least one place directive: {schedule_directives_file}")
    return n


def add_common_args(p: argparse.ArgumentParser, default_schedule: str) -> None:
    p.add_argument("--batch-size", type=int, default=4, help="micro-batch size (sequences per microbatch)")
    p.add_argument("--seq-len", type=int, default=1024)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--iters", type=int, default=3)
    p.add_argument("--iteration-sleep", type=float, default=0.0)
    p.add_argument("--activation-checkpointing", action="store_true", default=False)
    p.add_argument("--nsight", action="store_true", default=False, help="start every rank under `nsys profile` (one report per rank under <out-root>/nsight_reports)")
    p.add_argument("--viz", action="store_true", default=False, help="save schedule and per-rank DAG visualisations")
    p.add_argument("--temp-dir", default="/tmp/piper/tmp")
    p.add_argument("--use-inductor", action=argparse.BooleanOptionalAction, default=False,
                   help="accepted for compatibility; stage graphs always run the sm_100a kernels")
    p.add_argument("--pp-outer", action=argparse.BooleanOptionalAction, default=False,
                   help="accepted for compatibility; device ids in the schedule are used as given")
    p.add_argument("--schedule-directives-file", type=str, default=default_schedule)
    p.add_argument("--pytorch-profiler", action="store_true", default=False)
    p.add_argument("--pytorch-profiler-iters", type=int, default=3)
    p.add_argument("--device", default=None, choices=(None, "cuda", "cpu"))
    p.add_argument("--dtype", default="bf16", choices=("bf16", "fp32"))
    p.add_argument("--checkpoint-dir", default="", help="save a checkpoint here after the timed iterations")
    p.add_argument("--resume", default="", help="checkpoint directory to resume from")


def run_driver(args, model_class, model_args, cfg, loss_fn, const_attrs) -> dict:
    info_sched = load_schedule_directives(args.schedule_directives_file)
    from piper_b200.compiler.schedule import derive_schedule_info
    info = derive_schedule_info(info_sched, args.schedule_directives_file)
    mbs = int(info["num_microbatches"])
    rank = int(os.environ.get("RANK", "0"))
    g = torch.Generator().manual_seed(1234 + int(os.environ.get("PIPER_DP_RANK", "0")))
    x = torch.randint(0, cfg.vocab_size, (args.batch_size * mbs, args.seq_len), generator=g)
    y = torch.randint(0, cfg.vocab_size, (args.batch_size * mbs, args.seq_len), generator=g)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    actor = piper_setup(model_class, model_args=model_args, optim_fn=torch.optim.Adam, example_inputs=[x],
                        example_outputs=y, activation_checkpointing=args.activation_checkpointing,
                        num_checkpoints=getattr(args, "num_checkpoints", 1), model_dtype=dtype,
                        nsight=args.nsight, temp_dir=args.temp_dir, visualize_dag=args.viz, const_attrs=const_attrs,
                        use_inductor=args.use_inductor, pp_outer=args.pp_outer,
                        schedule_directives_file=args.schedule_directives_file, device=args.device,
                        artifact_dir=os.path.dirname(os.path.abspath(args.schedule_directives_file)))
    piper_metadata.tokens_per_step = args.batch_size * mbs * args.seq_len
    if args.resume:
        from piper_b200.runtime.checkpoint import load_checkpoint
        load_checkpoint(actor, args.resume)
    cuda = actor.device.type == "cuda"

    def timed_step(step_timeout=None):
        if cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            piper_exec_dag(loss_fn, log_stats=False, step_timeout=step_timeout)
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e) / 1e3
        t0 = time.perf_counter()
        piper_exec_dag(loss_fn, log_stats=False, step_timeout=step_timeout)
        return time.perf_counter() - t0

    logger.info(f"Running {args.warmup} warmup iterations")
    last = None
    for _ in range(args.warmup):
        last = timed_step()
        if args.iteration_sleep > 0:
            time.sleep(args.iteration_sleep)
    step_timeout = max(5.0, 5 * last) if last is not None else None
    logger.info(f"Running {args.iters} timed iterations")
    actor.reset_peak_memory()
    iter_times = []
    for _ in range(args.iters):
        iter_times.append(timed_step(step_timeout))
        if args.iteration_sleep > 0:
            time.sleep(args.iteration_sleep)
    peak = actor.get_and_reset_peak_memory_stats()
    if args.pytorch_profiler:
        prof_dir = getattr(args, "profile_dir", "") or os.path.join("out", "pytorch_profiles")
        actor.start_pytorch_profiler()
        for _ in range(args.pytorch_profiler_iters):
            piper_exec_dag(loss_fn, step_timeout=step_timeout)
        actor.stop_pytorch_profiler(prof_dir)
    if args.checkpoint_dir:
        from piper_b200.runtime.checkpoint import save_checkpoint
        save_checkpoint(actor, args.checkpoint_dir, step=actor.iteration,
                        schedule=piper_metadata.schedule_directives)
    return {
        "dp_rank": actor.layout.dp_rank, "pp_rank": actor.layout.pp_rank, "global_rank": rank, "model": args.model,
        "schedule": info.get("name"), "schedule_directives_file": args.schedule_directives_file,
        "pp": info.get("pp_degree"), "dp": info.get("dp_degree"), "batch_size": args.batch_size,
        "num_microbatches": mbs, "seq_len": args.seq_len, "iter_times_s": [float(t) for t in iter_times],
        "peak_memory_by_rank": {int(peak[0]): int(peak[1])},
        "losses": [float(v) for v in actor.last_losses],
    }
