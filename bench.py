"""Headline benchmark: training tokens/s of the Llama-3-8B-shape model, device-timed, max over ranks.

Usage (one rank per GPU, launched by torchrun for N > 1)::

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Work per step is fixed at 16 sequences of 4096 tokens (the PP4 x DP2 configuration's 2 x 8 microbatches of
1 x 4096), so scaling over N is strong scaling:

    N=1  PP1 x DP1, 16 microbatches        N=4  PP4 x DP1, 16 microbatches, 1F1B
    N=2  PP2 x DP1, 16 microbatches, 1F1B  N=8  PP4 x DP2, 8 microbatches per replica, 1F1B

Data is synthetic (uniform random tokens), weights are random-init N(0, 0.02), compute is bf16 with fp32
master weights and Adam state.  Two numbers are reported: ``value`` times K steps with the batch already on
the device; ``e2e`` times K further steps through the same public call with the step's tokens and labels
copied from pinned host memory and the loss read back to the host inside the timed region.  Every step's
inputs (64 Ki tokens), activations and the 16 GB of bf16 weights exceed the 126 MB L2 many times over.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PUBLISHED_TOKENS_PER_S = 13200.0   # "Piper eager, 1F1B" bar of the reference's figs/eval.png (hardware not stated)
SEQ = 4096
GLOBAL_SEQS = 16

LAYOUTS = {1: (1, 1), 2: (2, 1), 4: (4, 1), 8: (4, 2)}


def _schedule(n_gpus: int):
    from piper_b200.compiler.builders import build_1f1b_schedule

    pp, dp = LAYOUTS[n_gpus]
    mbs = GLOBAL_SEQS // dp
    sched = []
    for s in range(pp):
        devs = [s + pp * d for d in range(dp)]
        sched.append({"op": "place", "filter": {"PP": s}, "devices": devs, "stream": "pp_stream"})
    if dp > 1:
        for s in range(pp):
            devs = [s + pp * d for d in range(dp)]
            sched.append({"op": "replicate", "filter": {"PP": s}, "devices": devs, "reduce_stream": "dp_stream"})
    sched.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": mbs})
    sched += build_1f1b_schedule(pp, mbs)
    return sched, pp, dp, mbs


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from baseline.clocks import ClockSampler
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer, balanced_stage_layers
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.ops import native

    n = args.gpus
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    cfg = LLAMA_CONFIGS[args.model]
    sched, pp, dp, mbs = _schedule(n)
    g = torch.Generator().manual_seed(1234 + rank)
    tok = torch.randint(0, cfg.vocab_size, (mbs, SEQ + 1), generator=g)
    x_host, y_host = tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()
    split = balanced_stage_layers(cfg.n_layers, pp)
    actor = piper_setup(Transformer, (cfg, SEQ, pp, split), optim_fn=torch.optim.Adam, optim_kwargs={"lr": 1e-4},
                        example_inputs=[x_host], example_outputs=y_host, model_dtype=torch.bfloat16,
                        const_attrs=Transformer.const_attrs(cfg, SEQ), schedule_directives=sched, device="cuda",
                        no_nvtx=True)

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        piper_exec_dag(cross_entropy_loss)
    barrier()
    native.check_status()

    def timed(step_fn):
        sampler = ClockSampler(local)
        sampler.start()
        barrier()
        k0 = native.lib().kernel_launch_count()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        last = None
        for _ in range(args.steps):
            last = step_fn()
        e.record()
        barrier()
        ms = s.elapsed_time(e)
        launches = native.lib().kernel_launch_count() - k0
        clocks = sampler.stop()
        t = torch.tensor([ms], device="cuda")
        if n > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), launches, clocks, last

    ms_dev, launches, clocks, _ = timed(lambda: piper_exec_dag(cross_entropy_loss))

    def e2e_step():
        losses = piper_exec_dag(cross_entropy_loss, inputs=[x_host], labels=y_host)
        return [float(v) for v in losses]      # device -> host read of the step's result

    ms_e2e, _, _, last_losses = timed(e2e_step)
    host_ms = actor.last_host_time_s * 1e3
    node_times = None
    if os.environ.get("PIPER_BENCH_NODE_TIMES", "0") == "1":
        actor.time_nodes = True
        piper_exec_dag(cross_entropy_loss)
        node_times = {k: {kk: round(vv, 2) for kk, vv in v.items()} for k, v in actor.node_times.items()}
        actor.time_nodes = False
    native.check_status()
    tokens_per_step = GLOBAL_SEQS * SEQ
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    e2e_value = tokens_per_step * args.steps / (ms_e2e / 1e3)
    h2d = (x_host.numel() * x_host.element_size() if actor.has_first_stage() else 0) + \
          (y_host.numel() * y_host.element_size() if actor.has_loss_stage() else 0)
    d2h = 4 * len(last_losses or [])
    loss_sum, loss_cnt = float(sum(last_losses or [])), float(len(last_losses or []))
    if n > 1:
        # whole-job figures: bytes copied by every rank per step, mean loss over the ranks that hold a loss stage
        agg = torch.tensor([h2d, d2h, loss_sum, loss_cnt], device="cuda", dtype=torch.float64)
        dist.all_reduce(agg)
        h2d, d2h, loss_sum, loss_cnt = int(agg[0].item()), int(agg[1].item()), float(agg[2].item()), float(agg[3].item())
    return {
        "metric": "train tokens/sec (box, device-timed, max over ranks)", "value": value, "unit": "tokens/s",
        "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": value / PUBLISHED_TOKENS_PER_S,
        "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init N(0,0.02) weights",
        "config": {"model": f"llama3-{args.model}-shape", "global_batch": GLOBAL_SEQS, "seq_len": SEQ,
                   "num_microbatches": mbs, "parallelism": f"pp{pp}dp{dp}", "schedule": "1f1b", "stage_layers": split,
                   "optimizer": "Adam, fp32 master + moments", "l2": "per-step working set >> 126 MB L2"},
        "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "impl": "piper_b200", "loss": (loss_sum / loss_cnt) if loss_cnt else None,
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30, "host_ms_last_step": host_ms,
        "node_times_rank0": node_times,
    }


def run_reference(args) -> dict:
    from baseline.reference_arm import run as run_ref

    return run_ref(args)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--model", default="8b")
    args = ap.parse_args()
    if args.gpus not in LAYOUTS:
        raise SystemExit(f"--gpus must be one of {sorted(LAYOUTS)}")
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(out), flush=True)
    if args.impl == "reference":
        # the reference's actors own the process groups of this process (in other threads): leave without
        # running their destructors, which would wait for peers that have already left
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
