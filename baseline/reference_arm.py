"""``bench.py --impl reference``: the unmodified reference, run through its own public API.

The reference (installed with ``pip install --no-deps --target baseline/_ref``) is driven exactly as its
``examples/test_harness.py`` drives it: ``create_piper_placement_group`` -> ``PiperProgramCoordinator.run_program``
-> one ``run_dp_rank`` task per data-parallel replica -> ``piper_setup`` (its Dynamo backend, its directive
compiler, its ``PiperActor`` per GPU over NCCL) -> ``piper_exec_dag`` per step, on its own
``examples/models/llama3.py`` with eager PyTorch ops (``use_inductor=False``).  Nothing of ``piper_b200`` is
imported in these processes.

The reference needs Ray only as a transport for those calls.  When Ray is not installed, the stand-in under
``baseline/ray_shim`` maps them onto the processes this benchmark already has: one per GPU, started by
``torch.distributed.run`` (or the single ``python`` process for one GPU).  Process ``r`` hosts the actor with
global rank ``r``; the process that hosts pipeline rank 0 of a replica also runs that replica's driver task.

Timing: every actor process brackets the K timed steps with CUDA events on its own device (the reference ends
every step with a device synchronise); the reported time is the maximum over all actors.  The end-to-end figure
additionally re-loads the step's tokens and labels through ``PiperActor.load_input`` / ``load_labels`` (host to
device) every step and is timed on the host clock, as the reference's own examples time a step.

If the run fails (for example ``torch.OutOfMemoryError``: the reference's attention materialises S x S scores),
the arm prints ``{"impl": "reference", "unavailable": "<N and the error>"}`` and exits 0.
"""
from __future__ import annotations

import importlib.util
import json
import os
import sys
import tempfile
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SEQ = 4096
GLOBAL_SEQS = 16
LAYOUTS = {1: (1, 1), 2: (2, 1), 4: (4, 1), 8: (4, 2)}


def _setup_paths() -> None:
    for p in (os.path.join(REF, "examples"), REF):
        if p not in sys.path:
            sys.path.insert(0, p)
    if importlib.util.find_spec("ray") is None:
        sys.path.insert(0, os.path.join(HERE, "ray_shim"))


def _placement(kind, target, args, kwargs, options):
    """Which process hosts a new actor or task: actor of global rank r -> process r, replica driver -> its rank 0."""
    name = getattr(target, "__name__", "")
    if kind == "actor" and name == "PiperActor":
        return int(args[0]) + int(kwargs.get("dp_rank", 0)) * int(kwargs.get("pp_degree", 1))
    if kind == "task" and name == "run_dp_rank":
        dp_rank, _dp_degree, pp_degree = args[0], args[1], args[2]
        return int(dp_rank) * int(pp_degree)
    return None


def _write_schedule(path: str, pp: int, dp: int, mbs: int) -> None:
    """place / replicate / split directives plus the reference's own 1F1B order rows."""
    from build_schedule import build_1f1b_schedule      # baseline/_ref/examples/build_schedule.py

    sched = []
    for s in range(pp):
        sched.append({"op": "place", "filter": {"PP": s}, "devices": [s + pp * d for d in range(dp)],
                      "stream": "pp_stream"})
    if dp > 1:
        for s in range(pp):
            sched.append({"op": "replicate", "filter": {"PP": s}, "devices": [s + pp * d for d in range(dp)],
                          "reduce_stream": "dp_stream"})
    sched.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": mbs})
    sched += build_1f1b_schedule(pp, mbs)
    with open(path, "w") as f:
        json.dump(sched, f, indent=1)


# ---- functions that run inside an actor's thread (device timers) ---------------------------------------------
def _ev_start(actor):
    import torch

    torch.cuda.synchronize()
    actor._bench_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    actor._bench_events[0].record()
    return True


def _ev_stop(actor):
    import torch

    s, e = actor._bench_events
    e.record()
    torch.cuda.synchronize()
    return float(s.elapsed_time(e))


def _barrier(ray, key: str, n: int) -> None:
    """All ``n`` replica drivers meet here (a named counter actor, polled)."""
    if n <= 1:
        return

    class _Counter:
        def __init__(self):
            self.n = {}

        def arrive(self, k):
            self.n[k] = self.n.get(k, 0) + 1
            return self.n[k]

        def count(self, k):
            return self.n.get(k, 0)

    h = ray.remote(_Counter).options(name="piper_bench_barrier", get_if_exists=True, lifetime="detached").remote()
    ray.get(h.arrive.remote(key))
    deadline = time.monotonic() + 600
    while ray.get(h.count.remote(key)) < n:
        if time.monotonic() > deadline:
            raise TimeoutError(f"barrier {key}: not all {n} replica drivers arrived")
        time.sleep(0.002)


def _train(ns: dict, pg):
    """The training function handed to the reference's coordinator; mirrors ``examples/test_llama.py::main``."""
    import ray
    import torch
    from models.llama3 import LLAMA_8B, LLAMA_DEBUG, Transformer, precompute_freqs_cis
    from src.compile import piper_setup
    from src.piper import piper_exec_dag
    from src.state import piper_metadata

    cfg = {"8b": LLAMA_8B, "debug": LLAMA_DEBUG}[ns["model"]]
    seq, steps, warmup = ns["seq"], ns["steps"], ns["warmup"]
    dp_rank, dp = int(os.environ["PIPER_DP_RANK"]), int(os.environ["PIPER_DP_DEGREE"])
    loss_mod = torch.nn.CrossEntropyLoss()
    loss_fn = lambda output, labels: loss_mod(output.view(-1, output.size(-1)), labels.view(-1))  # noqa: E731

    g = torch.Generator().manual_seed(1234 + dp_rank)
    tok = torch.randint(0, cfg.vocab_size, (1, seq + 1), generator=g)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    freqs_cis = precompute_freqs_cis(cfg.dim // cfg.n_heads, seq, cfg.rope_theta)
    causal = torch.triu(torch.full((seq, seq), float("-inf")), diagonal=1)
    mask = torch.hstack([torch.zeros((seq, 0)), causal])

    piper_setup(Transformer, model_args=(cfg, seq), optim_fn=torch.optim.Adam, example_inputs=[x],
                example_outputs=y, model_dtype=torch.bfloat16, pg=pg, no_nvtx=True,
                const_attrs={"freqs_cis": freqs_cis, "mask": mask},
                use_inductor=bool(ns.get("use_inductor", False)),
                schedule_directives_file=ns["schedule"])
    actors = piper_metadata.actors
    handles = list(actors.values())
    loss_pp = max(actors.keys())
    for _ in range(warmup):
        piper_exec_dag(loss_fn)

    try:
        from ray._core import apply_on_actor
    except ImportError:          # real Ray: no hook into the actor process, host clock only
        apply_on_actor = None

    # K steps, device-timed on every actor
    _barrier(ray, "dev", dp)
    if apply_on_actor is not None:
        ray.get([apply_on_actor(a, _ev_start) for a in handles])
    t0 = time.perf_counter()
    for _ in range(steps):
        piper_exec_dag(loss_fn)
    wall_dev = (time.perf_counter() - t0) * 1e3
    dev_ms = ray.get([apply_on_actor(a, _ev_stop) for a in handles]) if apply_on_actor is not None else [wall_dev]

    # K more steps end to end: the step's tokens and labels go host -> device through the actors' loaders
    x_pin, y_pin = x.pin_memory() if torch.cuda.is_available() else x, y.pin_memory() if torch.cuda.is_available() else y
    _barrier(ray, "e2e", dp)
    t0 = time.perf_counter()
    n_losses = 0
    for _ in range(steps):
        ray.get(actors[0].load_input.remote([x_pin]))
        ray.get(actors[loss_pp].load_labels.remote(y_pin))
        n_losses = len(piper_exec_dag(loss_fn))
    e2e_ms = (time.perf_counter() - t0) * 1e3
    peaks = ray.get([a.get_and_reset_peak_memory_stats.remote() for a in handles])
    return {"dp_rank": dp_rank, "dev_ms": max(dev_ms), "wall_dev_ms": wall_dev, "e2e_ms": e2e_ms,
            "h2d": x.numel() * x.element_size() + y.numel() * y.element_size(), "d2h": 4 * n_losses,
            "peak_mem_gb": max(p[1] for p in peaks) / 2 ** 30}


def _error_line(n: int, exc: BaseException) -> str:
    text = " ".join(str(exc).split())
    note = " ".join(getattr(exc, "__notes__", []) or [])
    where = ""
    for line in note.splitlines():
        if "baseline/_ref/" in line and "File" in line:
            where = line.strip()
    return f"N={n}: {type(exc).__name__}: {text[:600]}" + (f" [{where}]" if where else "")


def run(args) -> dict | None:
    """Entry used by ``bench.py``.  Returns the JSON dict on process 0 and ``None`` on the other processes."""
    n = int(args.gpus)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if not os.path.isdir(os.path.join(REF, "src")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed on this box"} if rank == 0 else None
    if world != n:
        return {"impl": "reference", "unavailable": f"launched with {world} processes for --gpus {n}"} if rank == 0 else None
    _setup_paths()
    # the reference logs os.environ['CUDA_VISIBLE_DEVICES'] (Ray sets it); every process sees every GPU here
    import torch

    os.environ.setdefault("CUDA_VISIBLE_DEVICES", ",".join(str(i) for i in range(max(1, torch.cuda.device_count()))))
    # torch.distributed.run tells its workers that the launcher hosts their store; the reference's actors
    # rendezvous among themselves (tcp:// on a port of actor 0), where rank 0 has to start the server itself
    for var in ("TORCHELASTIC_USE_AGENT_STORE",):
        os.environ.pop(var, None)
    # a failed replica must not leave its peers bound to an NVLink multicast object
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import ray

    shim = hasattr(ray, "_core")
    if not shim and world > 1:
        return {"impl": "reference", "unavailable": "a real Ray is installed: use the reference's own harness"} \
            if rank == 0 else None
    rdv = os.path.join(tempfile.gettempdir(),
                       f"piper_ref_{os.environ.get('MASTER_PORT', '0')}_{os.getppid() if world > 1 else os.getpid()}")
    if shim:
        rt = ray._core.start(rank, world, rdv)
        ray._core.set_placement(_placement)
    if rank != 0:
        rt.serve_until_shutdown()
        return None

    pp, dp = LAYOUTS[n]
    if os.environ.get("PIPER_BENCH_LAYOUT"):           # smoke runs only
        pp, dp = (int(v) for v in os.environ["PIPER_BENCH_LAYOUT"].lower().split("x"))
    mbs = GLOBAL_SEQS // dp
    os.makedirs(rdv, exist_ok=True)
    sched_file = os.path.join(rdv, f"llama_pp{pp}_dp{dp}_1f1b_mbs{mbs}.json")
    result: dict = {}

    def job():
        try:
            from src.coordinator import PiperProgramCoordinator, create_piper_placement_group

            _write_schedule(sched_file, pp, dp, mbs)
            ray.init()
            pg = create_piper_placement_group(sched_file)
            ray.get(pg.ready(), timeout=600)
            coordinator = PiperProgramCoordinator.remote(schedule_directives_file=sched_file)
            ns = {"model": args.model, "seq": SEQ, "steps": int(args.steps), "warmup": int(args.warmup),
                  "schedule": sched_file, "use_inductor": os.environ.get("PIPER_REF_INDUCTOR", "0") == "1"}
            result["metrics"] = ray.get(coordinator.run_program.remote(_train, pg, ns, pg))
        except BaseException as exc:  # noqa: BLE001 - reported in the unavailable line
            result["error"] = exc

    from baseline.clocks import ClockSampler

    sampler = ClockSampler(list(range(n)))
    sampler.start()
    t = threading.Thread(target=job, daemon=True)
    t.start()
    t.join(float(os.environ.get("PIPER_REF_TIMEOUT_S", "1500")))
    clocks = sampler.stop()
    if shim:
        rt.shutdown_all()
    if t.is_alive():
        return {"impl": "reference", "unavailable": f"N={n}: no result after PIPER_REF_TIMEOUT_S seconds"}
    if "error" in result:
        return {"impl": "reference", "unavailable": _error_line(n, result["error"])}

    ms = result["metrics"]
    k = int(args.steps)
    dev_ms, e2e_ms = max(m["dev_ms"] for m in ms), max(m["e2e_ms"] for m in ms)
    tokens = GLOBAL_SEQS * SEQ
    return {
        "impl": "reference", "metric": "train tokens/sec (box, device-timed, max over ranks)",
        "value": tokens * k / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": n, "steps": k, "warmup": int(args.warmup),
        "ms_per_step": dev_ms / k, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init N(0,0.02) weights",
        "config": {"model": f"llama3-{args.model}-shape (reference examples/models/llama3.py)", "global_batch": GLOBAL_SEQS,
                   "seq_len": SEQ, "num_microbatches": mbs, "parallelism": f"pp{pp}dp{dp}", "schedule": "1f1b",
                   "stage_layers": "equal split (reference)", "optimizer": "torch.optim.Adam on bf16 parameters",
                   "use_inductor": os.environ.get("PIPER_REF_INDUCTOR", "0") == "1",
                   "transport": "ray stand-in over local sockets" if shim else "ray",
                   "l2": "per-step working set >> 126 MB L2"},
        "clocks": {**clocks, "note": "sampled over the whole run (compile, warm-up and timed steps)"},
        "e2e": {"value": tokens * k / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / k,
                "h2d_bytes_per_step": sum(m["h2d"] for m in ms), "d2h_bytes_per_step": sum(m["d2h"] for m in ms),
                "note": "host clock around load_input + load_labels + piper_exec_dag; the reference returns no loss"},
        "host_wall_ms_per_step": max(m["wall_dev_ms"] for m in ms) / k,
        "peak_mem_gb": max(m["peak_mem_gb"] for m in ms),
    }
