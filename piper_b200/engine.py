"""Compile driver and step driver: ``piper_setup`` and ``piper_exec_dag``.

``piper_setup`` has the keyword surface of the reference
(``src/compile.py:116-135``) but a different process model: there is no Ray
and no DAG shipping.  Every rank (one process per GPU, started by
``torchrun`` or by ``piper_b200.runtime.launcher``) loads the schedule,
traces the model on the ``meta`` device through the ``piper`` Dynamo backend,
runs the deterministic compiler, keeps the DAG of its own pipeline rank and
builds one local ``PiperActor`` from it.

``piper_exec_dag(loss_fn)`` runs one training step on the local actor and
returns this rank's per-microbatch losses.  ``step_timeout`` keeps the
reference's meaning (log that the step is overdue and keep waiting,
``src/piper.py:233-246``): the step runs on a worker thread and the caller
re-waits on it.
"""
from __future__ import annotations

import os
import threading
import time
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist

from . import api
from .compiler.dag import RECV, SEND, TrainingDAG
from .compiler.schedule import derive_schedule_info, load_schedule_directives, stage_device_map
from .runtime.actor import PiperActor
from .runtime.layout import ProcessGroups, RankLayout, init_distributed, make_layout
from .runtime.storage import AdamConfig
from .state import LOG_LEVEL, create_logger, piper_metadata

logger = create_logger("piper_engine", LOG_LEVEL)


def _pass_class(p: Optional[str]) -> str:
    return "F" if p == "F" else "B"


def assign_pipeline_channels(global_dag: TrainingDAG, per_device: list[TrainingDAG], layout_tuples: list) -> list:
    """Give every SEND/RECV pair its channel key and return the sorted list of all channels of the job.

    A channel is ``(sender rank, receiver rank, sender stage, receiver stage, pass class)``; the per-device DAGs
    store the rank-independent part and each rank substitutes its own data-parallel index.
    """
    bases = set()
    for n in global_dag.nodes.values():
        if n.node_kind != SEND:
            continue
        src, dst = global_dag.nodes[n.node_meta["from_uid"]], global_dag.nodes[n.node_meta["to_uid"]]
        base = (tuple(src.device), tuple(dst.device), int(src.tag.get("PP", src.node_meta.get("stage_id", 0)) or 0),
                int(dst.tag.get("PP", dst.node_meta.get("stage_id", 0)) or 0), _pass_class(src.tag.get("PASS")))
        bases.add(base)
        for uid in (n.uid, n.node_meta.get("pair_uid")):
            for sub in per_device:
                if uid in sub.nodes:
                    sub.nodes[uid].node_meta["channel_base"] = base
    channels = []
    for (sdev, ddev, fs, ts, pc) in sorted(bases):
        for i in range(len(sdev)):
            channels.append((sdev[i], ddev[i], fs, ts, pc))
    return sorted(channels)


def _bind_channels(dag: TrainingDAG, dp_rank: int) -> None:
    for n in dag.nodes.values():
        if n.node_kind in (SEND, RECV):
            sdev, ddev, fs, ts, pc = n.node_meta["channel_base"]
            n.node_meta["channel"] = (sdev[dp_rank], ddev[dp_rank], fs, ts, pc)


def _adam_config(optim_fn, optim_kwargs: Optional[dict]) -> AdamConfig:
    """Hyper-parameters of the flat Adam / AdamW kernels from the reference's ``optim_fn`` argument.

    The reference instantiates ``optim_class(params)`` per bucket (``src/actor.py:573,600``).  Here the update is
    one kernel over flat buffers, so only ``torch.optim.Adam`` (L2 decay added to the gradient) and
    ``torch.optim.AdamW`` (decoupled decay) can be honoured; ``optim_fn`` may be the class, a
    ``functools.partial`` of it, or ``None`` (Adam).  Anything the kernels cannot reproduce is rejected.
    """
    import functools

    kw: dict = {}
    fn = optim_fn
    while isinstance(fn, functools.partial):
        kw = {**fn.keywords, **kw}
        if fn.args:
            raise ValueError("optim_fn: positional arguments of a functools.partial are not supported")
        fn = fn.func
    kw.update(optim_kwargs or {})
    if fn is None:
        fn = torch.optim.Adam
    if fn not in (torch.optim.Adam, torch.optim.AdamW):
        raise ValueError(f"optim_fn={getattr(fn, '__name__', fn)!r}: the flat optimizer kernels implement "
                         "torch.optim.Adam and torch.optim.AdamW only")
    cfg = AdamConfig(decoupled=fn is torch.optim.AdamW)
    if fn is torch.optim.AdamW and "weight_decay" not in kw:
        cfg.weight_decay = 1e-2                     # torch.optim.AdamW's default
    for k, v in kw.items():
        if k == "lr":
            cfg.lr = float(v)
        elif k == "betas":
            cfg.betas = (float(v[0]), float(v[1]))
        elif k == "eps":
            cfg.eps = float(v)
        elif k == "weight_decay":
            cfg.weight_decay = float(v)
        elif k in ("fused", "foreach", "capturable", "differentiable"):
            continue                                # implementation switches of torch.optim, no effect on the math
        elif k in ("amsgrad", "maximize") and not v:
            continue
        else:
            raise ValueError(f"optimizer argument {k}={v!r} is not supported by the flat Adam/AdamW kernels")
    return cfg


def piper_setup(model_class, model_args=(), model_kwargs: Optional[dict] = None, optim_fn=None,
                example_inputs: Optional[list] = None, example_outputs=None, activation_checkpointing: bool = False,
                num_checkpoints: int = 1, model_dtype: torch.dtype = torch.bfloat16, use_inductor: bool = False,
                no_nvtx: bool = False, pg=None, nsight: bool = False, temp_dir: Optional[str] = None,
                visualize_dag: bool = False, const_attrs: Optional[dict] = None, pp_outer: bool = False,
                schedule_directives_file: Optional[str] = None, *, schedule_directives: Optional[list] = None,
                optim_kwargs: Optional[dict] = None, device: Optional[str] = None, seed: int = 0,
                artifact_dir: Optional[str] = None, baseline: Optional[str] = None,
                fused_collectives: Optional[bool] = None) -> PiperActor:
    """Compile ``model_class(*model_args)`` under the schedule and build this process's actor.

    ``example_inputs`` / ``example_outputs`` hold one replica's batch for a step (all microbatches
    concatenated on dim 0); they are loaded as the first step's data.  ``use_inductor``, ``pg``,
    ``temp_dir`` and ``pp_outer`` are accepted for call-site compatibility and have no effect: there is no
    Inductor/Triton path and no Ray placement group in this runtime.  ``nsight`` belongs to the launcher
    (``Coordinator(nsight=...)`` starts every rank under ``nsys profile``, the counterpart of the reference's
    per-actor ``runtime_env``, ``src/actor.py:57-64``); here it only checks that the process is being profiled.
    """
    del pg, temp_dir, pp_outer
    if nsight and not os.environ.get("NSYS_PROFILING_SESSION_ID"):
        logger.warning("nsight=True but this process does not run under nsys: start the job through "
                       "Coordinator(nsight=True) or the harness's --nsight")
    if model_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"model_dtype must be bfloat16 or float32, got {model_dtype}")
    if use_inductor:
        logger.info("use_inductor is ignored: stage graphs run the hand-written sm_100a kernels directly")
    if activation_checkpointing and num_checkpoints != 1:
        logger.info("activation checkpointing works per graph segment; num_checkpoints=%d is not used", num_checkpoints)
    torch._dynamo.reset()
    api._reset_annotation_state()

    if schedule_directives is None:
        if schedule_directives_file is None:
            raise ValueError("piper_setup needs schedule_directives_file or schedule_directives")
        schedule_directives = load_schedule_directives(schedule_directives_file)
    info = derive_schedule_info(schedule_directives, schedule_directives_file or "<inline>")
    piper_metadata.schedule_directives = schedule_directives
    piper_metadata.schedule_directives_file = schedule_directives_file
    piper_metadata.schedule_info = info
    piper_metadata.visualize_dag = visualize_dag
    if artifact_dir is not None:
        piper_metadata.artifact_dir = artifact_dir

    dev_type = device or ("cuda" if torch.cuda.is_available() else "cpu")
    stage_devs = stage_device_map(schedule_directives)
    world = len({d for t in stage_devs.values() for d in t})
    if world > 1 or dist.is_initialized():
        rank, ws, backend = init_distributed(dev_type)
        if ws != world:
            raise ValueError(f"schedule places {world} ranks but the job has WORLD_SIZE={ws}")
    else:
        rank, backend = min(d for t in stage_devs.values() for d in t), None
    layout = make_layout(stage_devs, rank, world)
    if dev_type == "cuda":
        dev = torch.device("cuda", torch.cuda.current_device())
    else:
        dev = torch.device("cpu")

    # --- trace on meta with the microbatch shape and compile ---------------------------------
    n_mbs = int(info["num_microbatches"])
    kwargs = {k: (v(info) if callable(v) else v) for k, v in (model_kwargs or {}).items()}
    with torch.device("meta"):
        model = model_class(*model_args, **kwargs)
    model = model.to(model_dtype) if model_dtype != torch.float32 else model
    meta_inputs = []
    for t in example_inputs or []:
        if isinstance(t, torch.Tensor):
            per = t.shape[0] // n_mbs if t.dim() > 0 and t.shape[0] % n_mbs == 0 and t.shape[0] >= n_mbs else t.shape[0]
            meta_inputs.append(torch.empty((per, *t.shape[1:]), dtype=t.dtype, device="meta"))
        else:
            meta_inputs.append(t)
    with torch._dynamo.config.patch(capture_scalar_outputs=True):
        compiled = torch.compile(model, backend="piper", fullgraph=True)
        with torch.no_grad():
            compiled(*meta_inputs)
    per_device = piper_metadata.per_pp_training_dags
    global_dag = piper_metadata.training_dag
    if per_device is None:
        raise RuntimeError("the piper backend did not run; is the model's forward traceable with fullgraph=True?")
    if len(per_device) != layout.pp_degree:
        raise RuntimeError(f"compiled {len(per_device)} per-device DAGs for {layout.pp_degree} pipeline ranks")
    channels = assign_pipeline_channels(global_dag, per_device, layout.device_tuples)
    if os.environ.get("PIPER_CHECK_PLANS", "1") != "0":
        # dispatch order, channel FIFO pairing and cross-rank deadlock freedom, checked on the host before launch
        from .compiler.check import check_plans
        check_plans(per_device)

    groups = None
    if backend is not None:
        groups = ProcessGroups(layout, backend)
        ep_groups = sorted({tuple(tuple(g) for g in n.node_meta["ep_shard"]["groups"])
                            for n in global_dag.nodes.values()
                            if n.node_meta.get("ep_shard") and n.node_meta["ep_shard"].get("groups")})
        for g in ep_groups:
            groups.ensure_ep_subgroups([list(x) for x in g])
        groups.declare_channels(channels)

    my_dag = per_device[layout.pp_rank]
    _bind_channels(my_dag, layout.dp_rank)
    actor = PiperActor(layout, groups, dev, model_dtype, _adam_config(optim_fn, optim_kwargs), seed=seed,
                       no_nvtx=no_nvtx, baseline=baseline or os.environ.get("PIPER_BASELINE"))
    actor.activation_checkpointing = bool(activation_checkpointing)
    actor.load_const_attrs(const_attrs or {})
    actor.load_training_dag(my_dag, n_mbs)
    if fused_collectives is None:
        fused_collectives = dev.type == "cuda" and actor.baseline != "nccl" and world > 1 \
            and os.environ.get("PIPER_FUSED", "1") != "0"
    if fused_collectives:
        from .parallel.fused import FusedCollectives
        actor.fused = FusedCollectives.create(actor)
    if dev.type == "cuda" and actor.baseline != "nccl" and os.environ.get("PIPER_FUSED", "1") != "0" \
            and (fused_collectives or os.environ.get("PIPER_FUSED_EP") == "force"):
        from .parallel.ep_fused import FusedExpertRuntime
        actor.ep_fused = FusedExpertRuntime.create(actor)
    if example_inputs is not None and actor.has_first_stage():
        actor.load_input(list(example_inputs))
    if example_outputs is not None and actor.has_loss_stage():
        actor.load_labels(example_outputs)
    piper_metadata.actors = {layout.pp_rank: actor}
    if example_inputs:
        t0 = example_inputs[0]
        if isinstance(t0, torch.Tensor) and t0.dim() >= 2:
            piper_metadata.tokens_per_step = int(t0.shape[0] * t0.shape[1])
    return actor


def piper_exec_dag(loss_fn: Callable, log_stats: bool = False, step_timeout: Optional[float] = None,
                   inputs: Optional[list] = None, labels=None) -> list:
    """Run one training step; returns this rank's per-microbatch losses (empty off the loss stage)."""
    actors = piper_metadata.actors
    if not actors:
        raise RuntimeError("piper_exec_dag called before piper_setup")
    t0 = time.perf_counter()
    results: list = []
    for actor in actors.values():
        if inputs is not None and actor.has_first_stage():
            actor.load_input(list(inputs))
        if labels is not None and actor.has_loss_stage():
            actor.load_labels(labels)
        if step_timeout is None:
            results.append(actor.run_dag(loss_fn))
            continue
        box: dict = {}

        def work(a=actor):
            try:
                if a.device.type == "cuda":
                    torch.cuda.set_device(a.device)
                box["out"] = a.run_dag(loss_fn)
            except BaseException as exc:   # re-raised on the caller's thread
                box["err"] = exc

        th = threading.Thread(target=work, daemon=True)
        th.start()
        while True:
            th.join(step_timeout)
            if not th.is_alive():
                break
            logger.warning(f"step exceeded step_timeout={step_timeout:.1f}s; "
                           "still waiting on in-flight step (peer may be down)")
        if "err" in box:
            raise box["err"]
        results.append(box["out"])
    step_time = time.perf_counter() - t0
    from .runtime.launcher import heartbeat
    heartbeat(next(iter(actors.values())).iteration)
    if log_stats:
        msg = [f"step_time={step_time:.3f}s"]
        if piper_metadata.tokens_per_step:
            msg.append(f"throughput={piper_metadata.tokens_per_step / step_time:.1f} tok/s")
        logger.info("  ".join(msg))
    losses: list = []
    for r in results:
        losses.extend(r.get("losses", []))
    return losses
