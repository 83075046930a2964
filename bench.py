"""Headline benchmark: training tokens/s, device-timed, max over ranks.

Usage (one rank per GPU, launched by torchrun for N > 1)::

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--config NAME]

``--config`` selects one of the four GPU configurations of the acceptance list (the default is the first):

``llama_pp4dp2`` (default)
    Llama-3-8B shape, 16 sequences of 4096 tokens per step whatever N (strong scaling):
    N=1 PP1, N=2 PP2, N=4 PP4 (16 microbatches, 1F1B), N=8 PP4 x DP2 (8 microbatches per replica, 1F1B, gradient
    buckets reduced by the fused reduce-scatter + Adam kernel under the remaining backward).
``llama_pp2dp4_zero3``
    Llama-3-8B shape, PP2 x DP4 with ZeRO-3 parameter and gradient sharding, 1F1B, 8 microbatches of 1 x 4096 per
    replica (N=8; N=4 runs PP2 x DP2).
``qwen_dualpipev``
    Qwen3-30B-A3B shape, four stages in V placement on two pipeline ranks x DP x EP, DualPipeV, 8 microbatches
    per replica.  N=8 uses DP4 with one expert-parallel group of 4 per pipeline rank, N=4 is DP2 x EP2.
``qwen_zero3_ep4``
    Qwen3-30B-A3B shape, PP2 x DP4 x EP4, ZeRO-3 for the non-expert parameters, 1F1B, 8 microbatches per replica.

Data is synthetic (uniform random tokens from one seeded stream, sliced per replica, labels = inputs shifted by
one), weights are random-init N(0, 0.02), compute is bf16 with fp32 master weights and Adam state.  Two numbers
are reported: ``value`` times K steps with the batch already on the device; ``e2e`` times K further steps through
the same public call with the step's tokens and labels copied from pinned host memory and the losses read back to
the host inside the timed region.  Every step's inputs, activations and the bf16 weights exceed the 126 MB L2
many times over, so nothing is flushed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

SEQ = 4096
CONFIGS = ("llama_pp4dp2", "llama_pp2dp4_zero3", "qwen_dualpipev", "qwen_zero3_ep4")
# (pipeline ranks, data-parallel degree) per config and GPU count
LAYOUTS = {
    "llama_pp4dp2": {1: (1, 1), 2: (2, 1), 4: (4, 1), 8: (4, 2)},
    "llama_pp2dp4_zero3": {2: (1, 2), 4: (2, 2), 8: (2, 4)},
    "qwen_dualpipev": {2: (1, 2), 4: (2, 2), 8: (2, 4)},
    "qwen_zero3_ep4": {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4)},
}
N1_RECORD = os.path.join(os.environ.get("TMPDIR", "/tmp"), "piper_bench_llama_pp4dp2_n1.json")


def _devices(s: int, pp: int, dp: int) -> list:
    return [s + pp * d for d in range(dp)]


def build_job(config: str, n_gpus: int, model: str, bucket_mb: int) -> dict:
    """Model, schedule directives and batch geometry of one benchmark configuration."""
    from piper_b200.compiler.builders import build_1f1b_schedule, build_dualpipev_schedule

    pp, dp = LAYOUTS[config][n_gpus]
    if os.environ.get("PIPER_BENCH_LAYOUT"):           # smoke runs only: "PPxDP" in place of the config's layout
        pp, dp = (int(v) for v in os.environ["PIPER_BENCH_LAYOUT"].lower().split("x"))
        if pp * dp != n_gpus:
            raise SystemExit(f"PIPER_BENCH_LAYOUT={pp}x{dp} does not use {n_gpus} GPUs")
    sched: list = []
    if config.startswith("llama"):
        from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer, balanced_stage_layers

        cfg = LLAMA_CONFIGS[model or "8b"]
        zero3 = config == "llama_pp2dp4_zero3"
        mbs = 8 if zero3 else 16 // dp
        split = balanced_stage_layers(cfg.n_layers, pp)
        for s in range(pp):
            sched.append({"op": "place", "filter": {"PP": s}, "devices": _devices(s, pp, dp), "stream": "pp_stream"})
        if dp > 1:
            for s in range(pp):
                rep = {"op": "replicate", "filter": {"PP": s}, "devices": _devices(s, pp, dp),
                       "reduce_stream": "dp_stream", "bucket_size": bucket_mb}
                if zero3:
                    rep.update({"gather_stream": "gather_stream", "shard_grads": True, "shard_params": True})
                sched.append(rep)
        sched.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": mbs})
        sched += build_1f1b_schedule(pp, mbs)
        return {"model_class": Transformer, "model_args": (cfg, SEQ, pp, split), "cfg": cfg, "sched": sched, "pp": pp,
                "dp": dp, "mbs": mbs, "const": Transformer.const_attrs(cfg, SEQ), "stage_layers": split,
                "model_name": f"llama3-{model or '8b'}-shape", "schedule": "1f1b",
                "parallelism": f"pp{pp}dp{dp}" + ("-zero3" if zero3 else "")}
    from piper_b200.models.qwen3 import QWEN3_CONFIGS, PiperQwen3Model

    import dataclasses

    # the configuration asks for a router that spreads tokens near-uniformly at initialisation: frozen-noise
    # top-k gating (see Qwen3Config.router_jitter_std)
    cfg = dataclasses.replace(QWEN3_CONFIGS[model or "30B-A3B"], router_jitter_std=8.0)
    mbs = 8
    v = config == "qwen_dualpipev"
    stages = 2 * pp if v else pp
    rank_of = (lambda s: s if s < pp else 2 * pp - 1 - s) if v else (lambda s: s)
    for s in range(stages):
        sched.append({"op": "place", "filter": {"PP": s}, "devices": _devices(rank_of(s), pp, dp), "stream": "pp_stream"})
    if dp > 1:
        for s in range(stages):
            rep = {"op": "replicate", "filter": {"PP": s}, "devices": _devices(rank_of(s), pp, dp),
                   "reduce_stream": "dp_stream"}
            if not v:
                rep.update({"gather_stream": "gather_stream", "shard_grads": True, "shard_params": True})
            sched.append(rep)
    for s in range(stages):
        sched.append({"op": "shard", "filter": {"PP": s, "EP": "*"}, "devices": _devices(rank_of(s), pp, dp),
                      "stream": "ep_stream"})
    sched.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": mbs})
    sched += build_dualpipev_schedule(pp, mbs) if v else build_1f1b_schedule(pp, mbs)
    return {"model_class": PiperQwen3Model, "model_args": (cfg, stages, SEQ), "cfg": cfg, "sched": sched, "pp": pp,
            "dp": dp, "mbs": mbs, "const": PiperQwen3Model.const_attrs(cfg, SEQ), "stage_layers": "equal split",
            "model_name": f"qwen3-{model or '30B-A3B'}-shape", "schedule": "dualpipev" if v else "1f1b",
            "parallelism": (f"pp{stages}(v on {pp} ranks)" if v else f"pp{pp}") + f"dp{dp}ep{dp}" + ("" if v else "-zero3")}


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from baseline.clocks import ClockSampler
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.ops import native

    n = args.gpus
    local = int(os.environ.get("LOCAL_RANK", "0"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(local)
    if args.config.startswith("qwen"):
        os.environ.setdefault("PIPER_EP_CAPACITY_FACTOR", "1.25")
        # the 30B shape is memory-tight: keep the host at most sixteen nodes (stage segments, exchanges)
        # ahead of the device so that blocks freed after a cross-stream use return to the allocator in time
        os.environ.setdefault("PIPER_MAX_RUN_AHEAD", "16")
    job = build_job(args.config, n, args.model, args.bucket_mb)
    cfg, pp, dp, mbs = job["cfg"], job["pp"], job["dp"], job["mbs"]
    global_seqs = dp * mbs
    # one token stream for the whole job: replica d trains on rows [d * mbs, (d + 1) * mbs) at every N, so the
    # printed loss is comparable across layouts
    g = torch.Generator().manual_seed(1234)
    tok = torch.randint(0, cfg.vocab_size, (global_seqs, SEQ + 1), generator=g)
    d = rank // pp
    mine = tok[d * mbs:(d + 1) * mbs]
    x_host, y_host = mine[:, :-1].contiguous().pin_memory(), mine[:, 1:].contiguous().pin_memory()

    def setup():
        return piper_setup(job["model_class"], job["model_args"], optim_fn=torch.optim.Adam,
                           optim_kwargs={"lr": 1e-4}, example_inputs=[x_host], example_outputs=y_host,
                           model_dtype=torch.bfloat16, const_attrs=job["const"], schedule_directives=job["sched"],
                           device="cuda", no_nvtx=True)

    actor = setup()

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps):
        sampler = ClockSampler(local)
        sampler.start()
        barrier()
        k0 = native.lib().kernel_launch_count()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        last = None
        for _ in range(steps):
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

    def run_all(a):
        for _ in range(args.warmup):
            piper_exec_dag(cross_entropy_loss)
        barrier()
        native.check_status()
        ms_dev, launches, clocks, _ = timed(lambda: piper_exec_dag(cross_entropy_loss), args.steps)
        tail = a.comm_tail_ms()
        return ms_dev, launches, clocks, tail

    ms_dev, launches, clocks, tail_ms = run_all(actor)

    def e2e_step():
        losses = piper_exec_dag(cross_entropy_loss, inputs=[x_host], labels=y_host)
        return [float(v) for v in losses]      # device -> host read of the step's result

    ms_e2e, _, _, last_losses = timed(e2e_step, args.steps)
    host_ms = actor.last_host_time_s * 1e3
    node_times = None
    if os.environ.get("PIPER_BENCH_NODE_TIMES", "0") == "1":
        actor.time_nodes = True
        piper_exec_dag(cross_entropy_loss)
        node_times = {k: {kk: round(vv, 2) for kk, vv in v.items()} for k, v in actor.node_times.items()}
        actor.time_nodes = False
    native.check_status()
    peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30
    fused = {"reduce_scatter_adam_buckets": len(actor.fused.buckets) if actor.fused else 0,
             "gather_gemm_buckets": sum(1 for b in actor.fused.buckets.values() if b.first_slot >= 0) if actor.fused else 0,
             "expert_exchange_slots": actor.ep_fused.slots if actor.ep_fused else 0}
    tokens_per_step = global_seqs * SEQ
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    e2e_value = tokens_per_step * args.steps / (ms_e2e / 1e3)
    h2d = (x_host.numel() * x_host.element_size() if actor.has_first_stage() else 0) + \
          (y_host.numel() * y_host.element_size() if actor.has_loss_stage() else 0)
    d2h = 4 * len(last_losses or [])
    loss_sum, loss_cnt = float(sum(last_losses or [])), float(len(last_losses or []))
    agg = torch.tensor([h2d, d2h, loss_sum, loss_cnt, tail_ms, peak_gb], device="cuda", dtype=torch.float64)
    if n > 1:
        # whole-job figures: bytes copied by every rank per step, mean loss over the ranks that hold a loss stage
        mx = agg[4:].clone()
        dist.all_reduce(agg)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        agg[4:] = mx
    h2d, d2h, loss_sum, loss_cnt = int(agg[0].item()), int(agg[1].item()), float(agg[2].item()), float(agg[3].item())
    tail_ms, peak_gb = float(agg[4].item()), float(agg[5].item())

    # the same DAG with every collective lowered to NCCL calls, for the fused-versus-NCCL end-to-end gain
    nccl_tps = None
    if args.nccl_arm and n > 1 and (actor.fused is not None or actor.ep_fused is not None) and peak_gb < 120:
        import gc

        from piper_b200.state import piper_metadata
        piper_metadata.actors = {}
        for rt in (actor.fused, actor.ep_fused):
            if rt is not None:
                rt.close()
        actor.fused = actor.ep_fused = None
        del actor
        gc.collect()
        torch.cuda.empty_cache()
        os.environ["PIPER_FUSED"] = "0"
        actor = setup()
        ms_nccl, _, _, _ = run_all(actor)
        nccl_tps = tokens_per_step * args.steps / (ms_nccl / 1e3)
        os.environ.pop("PIPER_FUSED", None)

    ms_step = ms_dev / args.steps
    sm = clocks.get("sm_mhz")
    cne = None
    if args.config == "llama_pp4dp2" and sm:
        # time x median SM clock separates layout efficiency from the clock a run happened to get: the N=1 run
        # of a scaling sweep leaves its figure where the larger runs of the same sweep can read it
        if rank == 0 and n == 1:
            try:
                with open(N1_RECORD, "w") as f:
                    json.dump({"ms_x_mhz": ms_step * sm}, f)
            except OSError:
                pass
        elif rank == 0 and os.path.exists(N1_RECORD):
            try:
                with open(N1_RECORD) as f:
                    cne = json.load(f)["ms_x_mhz"] / (n * ms_step * sm)
            except (OSError, ValueError, KeyError):
                cne = None
    return {
        "metric": "train tokens/sec (box, device-timed, max over ranks)", "value": value, "unit": "tokens/s",
        "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong" if args.config == "llama_pp4dp2" else "weak",
        "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init N(0,0.02) weights",
        "config": {"name": args.config, "model": job["model_name"], "global_batch": global_seqs, "seq_len": SEQ,
                   "num_microbatches": mbs, "parallelism": job["parallelism"], "schedule": job["schedule"],
                   "stage_layers": job["stage_layers"], "optimizer": "Adam, fp32 master + moments",
                   "bucket_size_mb": args.bucket_mb if dp > 1 else None,
                   **({"layout_override": os.environ["PIPER_BENCH_LAYOUT"]} if os.environ.get("PIPER_BENCH_LAYOUT") else {}),
                   "l2": "per-step working set >> 126 MB L2, no flush between steps"},
        "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "impl": "piper_b200", "loss": (loss_sum / loss_cnt) if loss_cnt else None,
        "peak_mem_gb": peak_gb, "host_ms_last_step": host_ms,
        "exposed_comm_ms": tail_ms, "ms_x_sm_mhz": (ms_step * sm) if sm else None,
        "clock_normalised_efficiency": cne, "nccl_lowering_tokens_per_s": nccl_tps, "fused_paths": fused,
        "node_times_rank0": node_times,
    }


def run_reference(args) -> dict:
    from baseline.reference_arm import run as run_ref

    if args.config != "llama_pp4dp2":
        return {"impl": "reference", "unavailable": f"config {args.config}: the reference arm runs the default "
                "configuration only (its Qwen example needs torchtitan.models.qwen3, which is not installed)"}
    return run_ref(args)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--config", default="llama_pp4dp2", choices=CONFIGS)
    ap.add_argument("--model", default=None, help="model size override (smaller shapes are for smoke runs only)")
    ap.add_argument("--bucket-mb", type=int, default=1000, help="replicate.bucket_size of the data-parallel buckets")
    ap.add_argument("--layout", default=None, help="PPxDP in place of the configuration's layout (smoke runs only)")
    ap.add_argument("--nccl-arm", action=argparse.BooleanOptionalAction, default=True,
                    help="also time the NCCL lowering of the same DAG (multi-GPU runs with a fused path)")
    args = ap.parse_args()
    if args.layout:
        os.environ["PIPER_BENCH_LAYOUT"] = args.layout
    if args.gpus not in LAYOUTS[args.config]:
        raise SystemExit(f"--gpus must be one of {sorted(LAYOUTS[args.config])} for --config {args.config}")
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    if args.impl == "reference":
        args.model = args.model or "8b"
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
