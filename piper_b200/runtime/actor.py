"""The per-GPU executor host (``PiperActor``) and its DAG executor.

One process owns one GPU and one ``PiperActor``.  The actor receives the
per-device training DAG of its pipeline rank, materialises the parameters of
every bucket it computes, and replays the DAG once per training step.  Task
semantics follow the reference interpreter (``src/executors.py:571-1003``):

========== ===============================================================
FWD        detach the inputs, run the segment's GraphModule, keep outputs
BWD        loss on the last segment, ``autograd.backward`` into the inputs
BWD_I      same with weight-gradient GEMMs queued instead of executed
BWD_W      drain that queue
SEND/RECV  one message per tensor on the channel's communicator
REDUCE     data-parallel gradient all-reduce (last microbatch of a bucket)
RS / AG    ZeRO reduce-scatter into the fp32 shard / parameter all-gather
A2A        expert-parallel token exchange (variable row counts)
UPD        optimizer step of every bucket, gradient reset
========== ===============================================================

What differs by design: microbatches are real slices of the step's batch and
the loss is the mean over the global batch; every cross-stream edge of the
DAG, temporal ones included, is enforced by a CUDA event rather than by host
issue order; pipeline receives land in buffers sized from the traced
shapes; per-microbatch losses are returned to the caller.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist
import torch.fx as fx

from ..compiler.dag import (A2A, ALL_GATHER, COMPUTE, DEFAULT_STREAM, ORDER_DUMMY, RECV, REDUCE, REDUCE_SCATTER, SEND,
                            UPD, TrainingDAG, TrainingDAGNode)
from ..compiler.ordering import serial_topological_order
from ..ops import core as ops_core
from ..ops import native
from ..state import LOG_LEVEL, create_logger
from .faults import FaultInjector
from .layout import ProcessGroups, RankLayout
from .storage import AdamConfig, ParamSlot, ParamStorage, init_tensor

logger = create_logger("piper_actor", LOG_LEVEL)


@dataclass
class StageBucket:
    """Everything needed to run one segment GraphModule: its placeholders and where their values come from."""
    key: str
    gm: fx.GraphModule
    n_placeholders: int
    input_pos: list                     # placeholder positions fed by runtime inputs, in order
    slots: list                         # ParamSlot per parameter/buffer placeholder
    storage: Optional[ParamStorage] = None
    constants: dict = field(default_factory=dict)    # placeholder position -> non-trainable tensor
    input_meta: list = field(default_factory=list)   # (shape, dtype) of the runtime inputs at trace time
    unsaved_outputs: Optional[list] = None           # output positions whose storage no backward formula keeps

    def build_args(self, inputs: list) -> list:
        args: list = [None] * self.n_placeholders
        for pos, t in zip(self.input_pos, inputs):
            args[pos] = t
        for pos, t in self.constants.items():
            args[pos] = t
        if self.storage is not None:
            if not self.storage.params_ready():
                raise RuntimeError(f"bucket {self.key}: parameters are sharded and were not gathered before use")
            for pos, t in self.storage.param_views.items():
                args[pos] = t
        missing = [i for i, a in enumerate(args) if a is None]
        if missing:
            raise RuntimeError(f"bucket {self.key}: placeholders {missing} have no value "
                               "(parameters not gathered, or an input is missing)")
        return args


class _Streams:
    """Logical stream name -> CUDA stream (or nothing on CPU)."""

    def __init__(self, device: torch.device, names: list[str]) -> None:
        self.cuda = device.type == "cuda"
        self.streams: dict[str, Any] = {}
        if self.cuda:
            for n in names:
                self.streams[n] = torch.cuda.current_stream(device) if n == DEFAULT_STREAM else torch.cuda.Stream(device)

    def get(self, name: str):
        return self.streams.get(name)

    def use(self, name: str):
        if not self.cuda:
            return _NullCtx()
        return torch.cuda.stream(self.streams[name])


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class PiperActor:
    """Owns the runtime state of one GPU: groups, streams, buckets, the DAG and its dispatch order."""

    def __init__(self, layout: RankLayout, groups: Optional[ProcessGroups], device: torch.device,
                 model_dtype: torch.dtype = torch.bfloat16, adam: Optional[AdamConfig] = None, seed: int = 0,
                 no_nvtx: bool = False, baseline: Optional[str] = None) -> None:
        self.layout = layout
        self.groups = groups
        self.device = device
        self.model_dtype = model_dtype
        self.adam = adam or AdamConfig()
        self.seed = seed
        self.no_nvtx = no_nvtx or device.type != "cuda"
        self.baseline = baseline            # "nccl": issue collectives exactly as the reference does
        self.dag: Optional[TrainingDAG] = None
        self.order: list[str] = []
        self.buckets: dict[str, StageBucket] = {}
        self.const_attrs: dict[str, torch.Tensor] = {}
        self.inputs: list = []
        self.labels: Optional[torch.Tensor] = None
        self.num_microbatches = 1
        self.iteration = 0
        self.faults = FaultInjector(layout.dp_rank)
        self.streams: Optional[_Streams] = None
        self.last_losses: list = []
        self.node_times: dict = {}
        self.profile_nodes = False
        self._profiler = None
        self.fused = None                   # parallel.fused.FusedCollectives when enabled
        self.ep_fused = None                # parallel.ep_fused.FusedExpertRuntime when enabled
        self._channel_streams: dict = {}
        self._ep_splits: dict = {}          # (MB, PP, EP) -> split sizes shared by a layer's four token exchanges
        self.time_nodes = False             # debug: CUDA-event and host time per DAG node kind, in node_times
        self.last_host_time_s = 0.0
        self.activation_checkpointing = False   # forward keeps segment inputs only; backward recomputes the segment
        self.debug_keep_grads = False       # tests: keep a scaled copy of the gradients each step
        self.drop_exchanged = os.environ.get("PIPER_DROP_EXCHANGED", "0") == "1"
        # kernels report expired waits and rejected indices through a per-device status word; it is read once
        # per step through pinned memory (no synchronisation) and a non-zero value of the previous step raises
        self.status_monitor = native.StatusMonitor(device) if device.type == "cuda" else None
        self.last_grads: dict = {}

    # ------------------------------------------------------------ loading
    def load_const_attrs(self, attrs: dict) -> None:
        for k, v in (attrs or {}).items():
            self.const_attrs[k] = v.to(self.device) if isinstance(v, torch.Tensor) else v

    def load_training_dag(self, dag: TrainingDAG, num_microbatches: int) -> None:
        self.dag = dag
        self.num_microbatches = num_microbatches
        names = sorted({n.stream for n in dag.nodes.values()} | {DEFAULT_STREAM})
        self.streams = _Streams(self.device, names)
        modes = self._bucket_modes(dag)
        for node in dag.nodes.values():
            if node.node_kind == COMPUTE and node.compute_subkind == "FWD":
                key = node.node_meta["bucket_key"]
                if key not in self.buckets:
                    self.buckets[key] = self._load_bucket(key, node, modes.get(key, "local"))
        self.order = serial_topological_order(dag)
        self._prune_redundant_grad_sync()
        computes = [u for u in self.order if dag.nodes[u].node_kind == COMPUTE]
        self._last_compute_uid = computes[-1] if computes else None
        self._tail_events = None
        self._plan = None
        self._release = None

    def _bucket_modes(self, dag: TrainingDAG) -> dict:
        modes: dict[str, str] = {}
        for n in dag.nodes.values():
            k = n.node_meta.get("bucket_key")
            if n.node_kind == ALL_GATHER:
                modes[k] = "zero3"
            elif n.node_kind == REDUCE_SCATTER and modes.get(k) != "zero3":
                modes[k] = "zero2"
            elif n.node_kind == REDUCE and k not in modes:
                modes[k] = "allreduce"
        return modes

    def _load_bucket(self, key: str, node: TrainingDAGNode, mode: str) -> StageBucket:
        m = node.node_meta
        gm: fx.GraphModule = m["gm"]
        _relocate_meta_devices(gm, self.device)
        phs = [n for n in gm.graph.nodes if n.op == "placeholder"]
        gargs = m["graphargs"]
        fqns = m.get("param_fqns") or [None] * len(phs)
        ep = m.get("ep_shard")
        ep_degree, ep_index = 1, 0
        if ep:
            ranks = _my_ep_ranks(ep, self.layout.global_rank)
            ep_degree, ep_index = len(ranks), ranks.index(self.layout.global_rank)
        slots, constants = [], {}
        for pos in m["param_idxs"]:
            g = gargs[pos]
            fqn = fqns[pos] if pos < len(fqns) and fqns[pos] else phs[pos].name
            trainable = bool(getattr(g, "requires_grad", False)) and g.is_floating_point()
            shape = tuple(g.shape)
            slot = ParamSlot(pos=pos, fqn=fqn, shape=shape, dtype=g.dtype, requires_grad=trainable)
            if ep and trainable and ep_degree > 1 and len(shape) >= 1 and shape[0] % ep_degree == 0:
                slot.ep_sharded, slot.full_shape = True, shape
                slot.ep_index, slot.ep_degree = ep_index, ep_degree
                slot.shape = (shape[0] // ep_degree, *shape[1:])
            if trainable:
                slots.append(slot)
            else:
                constants[pos] = self._constant_for(fqn, phs[pos].name, g)
        storage = None
        if slots:
            if mode != "local" and self.layout.dp_degree == 1:
                mode = "local"
            if ep and ep_degree > 1:
                mode = "local"          # experts are partitioned, not replicated: no data-parallel sync
            dtype = slots[0].dtype
            storage = ParamStorage(key, slots, self.device, dtype, mode, self.layout.dp_rank, self.layout.dp_degree,
                                   self.groups.dp_group if self.groups else None, self.adam, self.seed)
            if ep and ep_degree > 1 and ep.get("groups") and len(ep["groups"]) > 1 and self.groups is not None:
                # the same expert shard lives in every expert-parallel group: sum its gradients over those replicas
                storage.replica_group = self.groups.expert_replica_group
        input_meta = [(tuple(gargs[p].shape), gargs[p].dtype) for p in m["input_idxs"]]
        return StageBucket(key=key, gm=gm, n_placeholders=len(phs), input_pos=list(m["input_idxs"]), slots=slots,
                           storage=storage, constants=constants, input_meta=input_meta)

    def _constant_for(self, fqn: str, ph_name: str, meta_t: torch.Tensor) -> torch.Tensor:
        """Buffers and other non-trainable placeholders: taken from const_attrs by name, else zeros."""
        for k, v in self.const_attrs.items():
            if fqn == k or fqn.endswith("." + k) or k in ph_name:
                # the provided tensor keeps its dtype: rotary tables stay fp32 even when the module was cast to bf16
                return v.to(self.device)
        return torch.zeros(meta_t.shape, dtype=meta_t.dtype, device=self.device)

    def _prune_redundant_grad_sync(self) -> None:
        """Plain all-reduce buckets sync once per step: only the last REDUCE of a bucket does work."""
        last: dict[str, str] = {}
        for uid in self.order:
            n = self.dag.nodes[uid]
            if n.node_kind == REDUCE:
                last[n.node_meta.get("bucket_key")] = uid
        for uid in self.order:
            n = self.dag.nodes[uid]
            if n.node_kind == REDUCE:
                n.node_meta["noop"] = last[n.node_meta.get("bucket_key")] != uid
        # the last reduce-scatter of a bucket in a step is where the fused lowering applies the optimizer
        last_rs: dict[str, str] = {}
        for uid in self.order:
            n = self.dag.nodes[uid]
            if n.node_kind == REDUCE_SCATTER:
                last_rs[n.node_meta.get("bucket_key")] = uid
        for uid in self.order:
            n = self.dag.nodes[uid]
            if n.node_kind == REDUCE_SCATTER:
                n.node_meta["last_sync"] = last_rs[n.node_meta.get("bucket_key")] == uid

    # -------------------------------------------------------------- data
    def load_input(self, inputs: list) -> None:
        self.inputs = [t.to(self.device, non_blocking=True) if isinstance(t, torch.Tensor) else t for t in inputs]

    def load_labels(self, labels) -> None:
        self.labels = labels.to(self.device, non_blocking=True) if isinstance(labels, torch.Tensor) else labels

    def has_first_stage(self) -> bool:
        """True when some forward node takes the model inputs (no upstream segment, receive or exchange)."""
        for n in self.dag.nodes.values():
            if n.node_kind != COMPUTE or n.compute_subkind != "FWD":
                continue
            ups = [self.dag.nodes[p] for p in self.dag.data_preds(n.uid)]
            if not any(u.node_kind in (RECV, A2A) or (u.node_kind == COMPUTE and u.compute_subkind == "FWD")
                       for u in ups):
                return True
        return False

    def has_loss_stage(self) -> bool:
        return any(n.node_meta.get("compute_loss") for n in self.dag.nodes.values())

    # --------------------------------------------------------------- step
    def run_dag(self, loss_fn: Callable) -> dict:
        if self.device.type == "cuda" and not self.no_nvtx:
            torch.cuda.nvtx.range_push(f"iter_{self.iteration}_rank_{self.layout.global_rank}")
        if self.status_monitor is not None:
            self.status_monitor.poll()
        try:
            out = DagExecutor(self).run(loss_fn)
            if self.status_monitor is not None:
                self.status_monitor.post()
        finally:
            if self.device.type == "cuda" and not self.no_nvtx:
                torch.cuda.nvtx.range_pop()
        self.iteration += 1
        return out

    def native_plan(self, executor):
        """The C++ replay loop over this actor's dispatch order (built once); ``None`` selects the Python loop
        (``PIPER_NATIVE_EXECUTOR=0``, CPU runs, or the extension module is missing on a CPU-only machine)."""
        if self._plan is False:
            return None
        if self._plan is None:
            import os
            mod = _load_plan_module() if os.environ.get("PIPER_NATIVE_EXECUTOR", "1") != "0" else None
            if mod is None:
                if os.environ.get("PIPER_NATIVE_EXECUTOR", "1") != "0":
                    raise RuntimeError("the launch-plan executor piper_plan.so is missing; build it with "
                                       "`python -m piper_b200.build`")
                self._plan = False
                return None
            streams, node_stream, waits = executor.static_waits(self.order)
            labels = [_node_label(self.dag.nodes[u]) for u in self.order]
            self._plan_streams = streams          # keeps the torch stream objects alive
            self._plan = mod.PlanExecutor(self.device.index if self.device.index is not None else
                                          torch.cuda.current_device(), [int(s.cuda_stream) for s in streams],
                                          node_stream, waits, labels, not self.no_nvtx)
            self._plan.set_max_ahead(int(os.environ.get("PIPER_MAX_RUN_AHEAD", "0")))
        return self._plan

    def comm_tail_ms(self) -> float:
        """Device time of the last step between the end of its last compute node and the end of the step: the
        part of gradient synchronisation and optimizer work that no backward kernel was left to hide."""
        if self._tail_events is None:
            return 0.0
        e0, e1 = self._tail_events
        e1.synchronize()
        return float(e0.elapsed_time(e1))

    # ---------------------------------------------------- memory / profile
    def reset_peak_memory(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.reset_peak_memory_stats(self.device)

    def get_and_reset_peak_memory_stats(self) -> tuple[int, int]:
        peak = torch.cuda.max_memory_allocated(self.device) if self.device.type == "cuda" else 0
        self.reset_peak_memory()
        return self.layout.global_rank, int(peak)

    def start_pytorch_profiler(self) -> None:
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if self.device.type == "cuda" else [])
        self._profiler = profile(activities=acts)
        self._profiler.__enter__()
        self.profile_nodes = True

    def stop_pytorch_profiler(self, out_dir: str) -> str:
        import os
        self._profiler.__exit__(None, None, None)
        os.makedirs(out_dir, exist_ok=True)
        path = os.path.join(out_dir, f"dp{self.layout.dp_rank}_pp{self.layout.pp_rank}.json")
        self._profiler.export_chrome_trace(path)
        self._profiler, self.profile_nodes = None, False
        return path

    # ---------------------------------------------------------- parameters
    def named_parameters(self) -> dict[str, torch.Tensor]:
        """fqn -> full parameter tensor held by this rank (gathers ZeRO-3 shards)."""
        out = {}
        for b in self.buckets.values():
            if b.storage is None or b.storage.numel == 0:
                continue
            flat = b.storage.full_param_tensor()
            for s in b.storage.slots:
                out[s.fqn] = flat[s.offset:s.offset + s.numel].view(s.shape)
        return out

    def named_grads(self) -> dict[str, torch.Tensor]:
        out = {}
        for b in self.buckets.values():
            st = b.storage
            if st is None or st.flat_grads is None:
                continue
            for s in st.slots:
                out[s.fqn] = st.flat_grads[s.offset:s.offset + s.numel].view(s.shape)
        return out


def _node_label(node: TrainingDAGNode) -> str:
    tags = ",".join(f"{k}={v}" for k, v in sorted(node.tag.items(), key=lambda kv: kv[0]) if v is not None)
    return f"{node.node_kind}:{tags}:uid{node.uid}"


def _load_plan_module():
    """The C++ launch-plan executor (``csrc/plan/plan_executor.cpp``), built next to the kernel library."""
    import importlib.util

    path = native.lib_path().with_name("piper_plan.so")
    if not path.exists():
        return None
    spec = importlib.util.spec_from_file_location("piper_plan", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _my_ep_ranks(ep: dict, rank: int) -> list:
    groups = ep.get("groups")
    if groups:
        for g in groups:
            if rank in g:
                return list(g)
    return list(ep["devices"])


def _relocate_meta_devices(gm: fx.GraphModule, device: torch.device) -> None:
    """Graphs are traced on ``meta``; device literals baked into factory calls must point at the real device."""
    changed = False
    for n in gm.graph.nodes:
        if n.op in ("call_function", "call_method") and "device" in n.kwargs:
            d = n.kwargs["device"]
            if (isinstance(d, torch.device) and d.type == "meta") or d == "meta":
                kw = dict(n.kwargs)
                kw["device"] = device
                n.kwargs = kw
                changed = True
        new_args = tuple(device if (isinstance(a, torch.device) and a.type == "meta") else a for a in n.args)
        if new_args != tuple(n.args):
            n.args = new_args
            changed = True
    if changed:
        gm.recompile()


class DagExecutor:
    """Replays the actor's dispatch order once: one training step."""

    def __init__(self, actor: PiperActor) -> None:
        self.a = actor
        self.dag = actor.dag
        self.cuda = actor.device.type == "cuda"
        self.events: dict[str, Any] = {}
        self.fwd_ctx: dict[str, tuple] = {}      # fwd uid -> (detached inputs, outputs)
        self.outs: dict[str, Any] = {}           # producer uid -> tuple of tensors for data successors
        self.pending: list = []                  # async send/recv work handles
        self.wgrad_queues: dict[str, list] = {}
        self.shape_ref: dict[str, list] = {}
        self.losses: list = []

    # ----------------------------------------------------------- helpers
    def _mb(self, node: TrainingDAGNode) -> int:
        v = node.tag.get("MB", 0)
        return int(v) if v is not None else 0

    def _microbatch(self, t, mb: int):
        if not isinstance(t, torch.Tensor) or t.dim() == 0:
            return t
        n = self.a.num_microbatches
        if t.shape[0] % n == 0 and t.shape[0] >= n:
            per = t.shape[0] // n
            return t[mb * per:(mb + 1) * per]
        return t

    def _stream(self, node: TrainingDAGNode):
        """CUDA stream a node runs on.  Pipeline messages get one stream per channel, so a send that waits for
        its peer never blocks a receive of another channel queued behind it."""
        if node.node_kind in (SEND, RECV):
            key = tuple(node.node_meta.get("channel") or ())
            st = self.a._channel_streams.get(key)
            if st is None:
                st = self.a._channel_streams[key] = torch.cuda.Stream(self.a.device)
            return st
        return self.a.streams.get(node.stream)

    def _wait_preds(self, node: TrainingDAGNode) -> None:
        if not self.cuda:
            return
        s = self._stream(node)
        p2p = node.node_kind in (SEND, RECV)
        for e in self.dag.in_edges(node.uid):
            p = e.src_uid
            pn = self.dag.nodes[p]
            if p not in self.events:
                continue
            # order between pipeline messages is host issue order only; an event wait on a send that is
            # itself waiting for the peer could stall a receive the peer needs first
            if p2p and pn.node_kind in (SEND, RECV) and e.dep_kind == "temporal":
                continue
            ev, ps = self.events[p]
            if ps is not s:
                s.wait_event(ev)

    def _record(self, node: TrainingDAGNode) -> None:
        if self.cuda:
            s = self._stream(node)
            ev = torch.cuda.Event()
            ev.record(s)
            self.events[node.uid] = (ev, s)

    def _inputs_for(self, node: TrainingDAGNode) -> list:
        """Runtime inputs of a forward node: outputs of the previous segment, a receive or an exchange buffer,
        or (first segment) this microbatch's slice of the step's model inputs."""
        for p in self.dag.data_preds(node.uid):
            pn = self.dag.nodes[p]
            if p in self.outs and (pn.node_kind in (RECV, A2A)
                                   or (pn.node_kind == COMPUTE and pn.compute_subkind == "FWD")):
                self._wait_work(p)
                return list(self.outs[p])
        return [self._microbatch(t, self._mb(node)) for t in self.a.inputs]

    def _wait_work(self, uid: str) -> None:
        for w in self._works.pop(uid, []):
            w.wait()

    def _release_plan(self) -> tuple:
        """Static lifetime of every node's outputs: ``release[i]`` lists the producers whose last reader is node
        ``i`` of the dispatch order, ``readers[p]`` the nodes that read producer ``p``.  Without it every gradient
        tuple, receive buffer and exchange result of a step would stay referenced until the step ends."""
        a = self.a
        if a._release is None:
            index = {u: i for i, u in enumerate(a.order)}
            last: dict[str, int] = {}
            readers: dict[str, list] = {}
            for i, u in enumerate(a.order):
                n = self.dag.nodes[u]
                reads = set(self.dag.data_preds(u))
                reads.add(n.node_meta.get("from_uid"))
                reads.add(n.node_meta.get("fwd_uid"))
                for p in reads:
                    if p in index and p != u:
                        last[p] = max(last.get(p, -1), i)
                        readers.setdefault(p, []).append(u)
            release: list[list] = [[] for _ in a.order]
            for p, i in last.items():
                release[i].append(p)
            for u, i in index.items():
                if u not in last:
                    release[i].append(u)               # read by nobody (gradients of the model inputs)
                    readers[u] = []
            a._release = (release, readers)
        return a._release

    def _release_outputs(self, i: int) -> None:
        """Drop the outputs whose last reader was node ``i``.  A block that another stream has read goes back to
        its own stream's pool only after that stream has passed the read."""
        release, readers = self._release_plan()
        for p in release[i]:
            vals = self.outs.pop(p, None)
            if not vals or not self.cuda:
                continue
            ps = self._stream(self.dag.nodes[p])
            others = {id(s): s for s in (self._stream(self.dag.nodes[u]) for u in readers[p]) if s is not ps}
            for t in vals:
                if isinstance(t, torch.Tensor) and t.is_cuda:
                    for s in others.values():
                        t.record_stream(s)

    # --------------------------------------------------------------- run
    def run(self, loss_fn: Callable) -> dict:
        a = self.a
        self._works: dict[str, list] = {}
        t0 = time.perf_counter()
        timed: list = []
        if self.cuda:
            # side streams must see the previous step's update before they touch parameters again
            cur = a.streams.get(DEFAULT_STREAM)
            for name, s in a.streams.streams.items():
                if name != DEFAULT_STREAM:
                    s.wait_stream(cur)
            for s in a._channel_streams.values():
                s.wait_stream(cur)
        self._tail0 = None
        plan = a.native_plan(self) if (self.cuda and not a.profile_nodes) else None
        if plan is not None:
            # the C++ executor owns stream switching, event waits/records, NVTX ranges and per-node timing;
            # Python only runs the bodies
            nodes = [self.dag.nodes[uid] for uid in a.order]
            host_ms = [0.0] * len(nodes) if a.time_nodes else None
            plan.set_timing(bool(a.time_nodes))

            def body(i: int) -> None:
                t_node = time.perf_counter() if host_ms is not None else 0.0
                self._dispatch(nodes[i], loss_fn)
                self._release_outputs(i)
                if host_ms is not None:
                    host_ms[i] = (time.perf_counter() - t_node) * 1e3

            plan.run(body)
            if a.time_nodes:
                dev_ms = plan.elapsed()
                timed = [(n.uid, n.compute_subkind or n.node_kind, dev_ms[i], host_ms[i]) for i, n in enumerate(nodes)]
        else:
            for pos, uid in enumerate(a.order):
                node = self.dag.nodes[uid]
                label = None
                if self.cuda and (not a.no_nvtx or a.profile_nodes):
                    label = _node_label(node)
                    if not a.no_nvtx:
                        torch.cuda.nvtx.range_push(label)
                rf = torch.profiler.record_function(label) if (a.profile_nodes and label) else _NullCtx()
                with rf, (torch.cuda.stream(self._stream(node)) if self.cuda else _NullCtx()):
                    self._wait_preds(node)
                    t_node = time.perf_counter()
                    if a.time_nodes and self.cuda:
                        ev0 = torch.cuda.Event(enable_timing=True)
                        ev0.record(self._stream(node))
                    self._dispatch(node, loss_fn)
                    self._record(node)
                    self._release_outputs(pos)
                    if a.time_nodes:
                        host = (time.perf_counter() - t_node) * 1e3
                        if self.cuda:
                            ev1 = torch.cuda.Event(enable_timing=True)
                            ev1.record(self._stream(node))
                            timed.append((uid, node.compute_subkind or node.node_kind, (ev0, ev1), host))
                        else:
                            timed.append((uid, node.compute_subkind or node.node_kind, None, host))
                if label is not None and not a.no_nvtx:
                    torch.cuda.nvtx.range_pop()
        for ws in self._works.values():
            for w in ws:
                w.wait()
        for w in self.pending:
            w.wait()
        if self.cuda:
            # later steps reuse buffers on the default stream: fence the side streams behind it
            cur = a.streams.get(DEFAULT_STREAM)
            for name, s in a.streams.streams.items():
                if name != DEFAULT_STREAM:
                    cur.wait_stream(s)
            for s in a._channel_streams.values():
                cur.wait_stream(s)
            if self._tail0 is not None:
                tail1 = torch.cuda.Event(enable_timing=True)
                tail1.record(cur)
                a._tail_events = (self._tail0, tail1)
        a.last_losses = self.losses
        host_s = time.perf_counter() - t0
        a.last_host_time_s = host_s
        if a.time_nodes:
            if self.cuda:
                torch.cuda.synchronize()
            per_kind: dict = {}
            for uid, k, dev, host in timed:
                rec = per_kind.setdefault(k, {"count": 0, "device_ms": 0.0, "host_ms": 0.0})
                rec["count"] += 1
                rec["host_ms"] += host
                if isinstance(dev, tuple):
                    rec["device_ms"] += dev[0].elapsed_time(dev[1])
                elif dev is not None:
                    rec["device_ms"] += float(dev)
            a.node_times = per_kind
        return {"losses": self.losses, "host_time_s": host_s}

    def _dispatch(self, node: TrainingDAGNode, loss_fn: Callable) -> None:
        """Body of one node; the caller has made the node's stream current and enqueued its event waits."""
        a = self.a
        kind = node.node_kind
        if kind == COMPUTE:
            sub = node.compute_subkind
            if sub == "FWD":
                self._forward(node)
            elif sub == "BWD":
                a.faults.maybe_fire("bwd", a.iteration)
                self._backward(node, loss_fn, split=False)
            elif sub == "BWD_I":
                a.faults.maybe_fire("bwd", a.iteration)
                self._backward(node, loss_fn, split=True)
            elif sub == "BWD_W":
                self._backward_weight(node)
        elif kind == SEND:
            self._send(node)
        elif kind == RECV:
            self._recv(node)
        elif kind == REDUCE:
            self._all_reduce(node)
        elif kind == REDUCE_SCATTER:
            self._reduce_scatter(node)
        elif kind == ALL_GATHER:
            self._all_gather(node)
        elif kind == A2A:
            self._all_to_all(node)
        elif kind == UPD:
            self._update(node)
        if self.cuda and node.uid == a._last_compute_uid:
            self._tail0 = torch.cuda.Event(enable_timing=True)
            self._tail0.record(self._stream(node))

    def static_waits(self, order: list) -> tuple:
        """The plan behind ``_wait_preds``: per node the stream it runs on and the earlier nodes on other streams
        that it waits for (order between pipeline messages is host issue order only)."""
        index = {uid: i for i, uid in enumerate(order)}
        streams, stream_ids, node_stream, waits = [], {}, [], []
        for uid in order:
            s = self._stream(self.dag.nodes[uid])
            if id(s) not in stream_ids:
                stream_ids[id(s)] = len(streams)
                streams.append(s)
            node_stream.append(stream_ids[id(s)])
        for i, uid in enumerate(order):
            node = self.dag.nodes[uid]
            p2p = node.node_kind in (SEND, RECV)
            w = set()
            for e in self.dag.in_edges(uid):
                j = index.get(e.src_uid)
                if j is None or j >= i:
                    continue
                pn = self.dag.nodes[e.src_uid]
                if p2p and pn.node_kind in (SEND, RECV) and e.dep_kind == "temporal":
                    continue
                if node_stream[j] != node_stream[i]:
                    w.add(j)
            waits.append(sorted(w))
        return streams, node_stream, waits

    # ------------------------------------------------------------ compute
    def _forward(self, node: TrainingDAGNode) -> None:
        a = self.a
        bucket = a.buckets[node.node_meta["bucket_key"]]
        raw = self._inputs_for(node)
        ins = []
        for t in raw:
            if isinstance(t, torch.Tensor):
                t = t.detach()
                if t.is_floating_point():
                    t.requires_grad_(True)
            ins.append(t)
        if a.ep_fused is not None:
            a.ep_fused.enter(node)
        try:
            if a.activation_checkpointing:
                # keep only the segment's inputs; the backward node re-runs the segment with autograd on
                with torch.no_grad():
                    outs = bucket.gm(*bucket.build_args(ins))
            elif bucket.unsaved_outputs is None and (a.drop_exchanged or not self.cuda):
                outs = self._forward_tracking_saved(bucket, ins)
            else:
                outs = bucket.gm(*bucket.build_args(ins))
        finally:
            if a.ep_fused is not None:
                a.ep_fused.leave()
        outs = tuple(outs) if isinstance(outs, (tuple, list)) else (outs,)
        self.fwd_ctx[node.uid] = (ins, None if a.activation_checkpointing else outs)
        self.outs[node.uid] = outs
        self.shape_ref[node.uid] = [(tuple(o.shape), o.dtype) for o in outs
                                    if isinstance(o, torch.Tensor) and o.is_floating_point()]
        if node.node_meta.get("zero_free_full_params_after") and bucket.storage is not None:
            self._free_params(bucket.storage, node)

    @staticmethod
    def _forward_tracking_saved(bucket: StageBucket, ins: list):
        """First run of a segment: note which outputs no backward formula saved (directly or through a view) and
        which do not alias an input.  Such an output is needed after the forward pass only by whoever reads it,
        so its memory can go once an exchange has copied it away (``_drop_exchanged``)."""
        saved: set = set()

        def pack(t):
            if isinstance(t, torch.Tensor) and t.device.type != "meta":
                saved.add(t.untyped_storage().data_ptr())
            return t

        with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
            outs = bucket.gm(*bucket.build_args(ins))
        seq = tuple(outs) if isinstance(outs, (tuple, list)) else (outs,)
        held = saved | {t.untyped_storage().data_ptr() for t in ins if isinstance(t, torch.Tensor)}
        bucket.unsaved_outputs = [i for i, o in enumerate(seq) if isinstance(o, torch.Tensor) and o.numel() > 0
                                  and o.untyped_storage().data_ptr() not in held]
        return outs

    def _drop_exchanged(self, src: str, node: TrainingDAGNode, vals: list, res: tuple) -> None:
        """The exchanged tensor of a forward segment has been copied to its destination: if the exchange is the
        segment's only reader and no backward formula kept the tensor, give its memory back now instead of at the
        segment's backward pass (the tensor object stays as the root of the backward call).

        On CUDA devices this is opt-in (``PIPER_DROP_EXCHANGED=1``): it has only been validated on CPU ranks."""
        if self.cuda and not self.a.drop_exchanged:
            return
        pn = self.dag.nodes[src]
        ctx = self.fwd_ctx.get(src)
        if not (pn.node_kind == COMPUTE and pn.compute_subkind == "FWD") or ctx is None or ctx[1] is None:
            return
        bucket = self.a.buckets[pn.node_meta["bucket_key"]]
        ti = node.node_meta.get("a2a_tensor_idx")
        if ti is None or bucket.unsaved_outputs is None or ti not in bucket.unsaved_outputs:
            return
        _release, readers = self._release_plan()
        forward_readers = [u for u in readers.get(src, [])
                           if not (self.dag.nodes[u].node_kind == COMPUTE and self.dag.nodes[u].compute_subkind != "FWD")]
        t, r = vals[ti], res[ti]
        if forward_readers != [node.uid] or not isinstance(t, torch.Tensor) or not isinstance(r, torch.Tensor):
            return
        if r.untyped_storage().data_ptr() == t.untyped_storage().data_ptr() or not t.untyped_storage().resizable():
            return                                    # passed through (a group of one rank), or memory of a fixed buffer
        if t.is_cuda:
            t.record_stream(self._stream(node))
        t.untyped_storage().resize_(0)

    def _output_grads(self, node: TrainingDAGNode):
        """Gradients w.r.t. this segment's outputs from the downstream backward / receive / exchange node.

        Returns ``(grads, compact)``; ``compact`` is True for a pipeline receive, whose list has one entry per
        floating-point output instead of one per output.
        """
        for p in self.dag.data_preds(node.uid):
            pn = self.dag.nodes[p]
            if p not in self.outs:
                continue
            if pn.node_kind in (RECV, A2A) or (pn.node_kind == COMPUTE and pn.compute_subkind in ("BWD", "BWD_I")):
                self._wait_work(p)
                return list(self.outs[p]), pn.node_kind == RECV
        return None, False

    def _backward(self, node: TrainingDAGNode, loss_fn: Callable, split: bool) -> None:
        a = self.a
        fwd_uid = node.node_meta["fwd_uid"]
        bucket = a.buckets[node.node_meta["bucket_key"]]
        st = bucket.storage
        if st is not None and node.node_meta.get("zero_alloc_full_grads_before"):
            st.alloc_grads()
        ins, outs = self.fwd_ctx.pop(fwd_uid)
        self.outs.pop(fwd_uid, None)
        if outs is None:
            # activation checkpointing: rebuild the autograd graph of this segment from its saved inputs
            if a.ep_fused is not None:
                a.ep_fused.enter(self.dag.nodes[fwd_uid], replay=True)
            try:
                outs = bucket.gm(*bucket.build_args(ins))
            finally:
                if a.ep_fused is not None:
                    a.ep_fused.leave()
            outs = tuple(outs) if isinstance(outs, (tuple, list)) else (outs,)
        if split:
            ops_core.wgrad_store.begin()
        join_scope = ops_core.deferred_join()
        join_scope.__enter__()
        try:
            if node.node_meta.get("compute_loss"):
                labels = self._microbatch(a.labels, self._mb(node))
                loss = loss_fn(outs[0], labels)
                self.losses.append(loss.detach())
                loss.backward()
            else:
                grads, compact = self._output_grads(node)
                if grads is None:
                    raise RuntimeError(f"{node.uid}: no upstream gradient available")
                if compact:
                    # received over a pipeline channel: one gradient per floating-point output, in order
                    it = iter(grads)
                    grads = [next(it) if isinstance(o, torch.Tensor) and o.is_floating_point() else None
                             for o in outs]
                pairs = [(o, g) for o, g in zip(outs, grads)
                         if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
                if pairs:
                    torch.autograd.backward([p[0] for p in pairs], [p[1] for p in pairs])
        finally:
            join_scope.__exit__(None, None, None)
            if split:
                self.wgrad_queues[node.uid] = ops_core.wgrad_store.end()
        # one slot per input; a floating-point input that received no gradient reports zeros, so that both ends
        # of a pipeline channel agree on "one message per floating-point tensor"
        in_grads = tuple((t.grad if t.grad is not None else torch.zeros_like(t))
                         if isinstance(t, torch.Tensor) and t.is_floating_point() else None for t in ins)
        self.outs[node.uid] = in_grads
        if st is not None and st.flat_grads is not None:
            st.absorb_autograd_grads()
        if not split and node.node_meta.get("zero_free_full_params_after") and st is not None:
            self._free_params(st, node)
        if a.ep_fused is not None:
            a.ep_fused.after_node(node)

    def _backward_weight(self, node: TrainingDAGNode) -> None:
        a = self.a
        bucket = a.buckets[node.node_meta["bucket_key"]]
        st = bucket.storage
        bi_uid = next((p for p in self.dag.data_preds(node.uid)
                       if self.dag.nodes[p].node_kind == COMPUTE and self.dag.nodes[p].compute_subkind == "BWD_I"), None)
        queue = self.wgrad_queues.pop(bi_uid, []) if bi_uid else []
        if st is not None and node.node_meta.get("zero_alloc_full_grads_before"):
            st.alloc_grads()
        for w, dw in ops_core.WgradStore.drain(queue):
            sink = ops_core.grad_sinks.get(w)
            if sink is not None:
                sink.add_(dw.to(torch.float32))
            elif w.grad is None:
                w.grad = dw
            else:
                w.grad.add_(dw)
        if st is not None and st.flat_grads is not None:
            st.absorb_autograd_grads()
        if node.node_meta.get("zero_free_full_params_after") and st is not None:
            self._free_params(st, node)
        if a.ep_fused is not None:
            a.ep_fused.after_node(node)

    # ---------------------------------------------------- communication
    def _channel(self, node: TrainingDAGNode):
        key = node.node_meta.get("channel")
        if key is None:
            raise RuntimeError(f"{node.uid}: pipeline channel was not assigned")
        return self.a.groups.channel(tuple(key))

    def _send(self, node: TrainingDAGNode) -> None:
        a = self.a
        src = node.node_meta["from_uid"]
        vals = self.outs.get(src)
        if vals is None:
            raise RuntimeError(f"{node.uid}: nothing to send from {src}")
        peer = a.layout.peer_rank(node.node_meta["peer_pp_rank"])
        group, tag = self._channel(node)
        tensors = [t.detach().contiguous() for t in vals if isinstance(t, torch.Tensor)]
        if self.cuda and len(tensors) > 1:
            # all tensors of a stage boundary go out as one grouped NCCL call
            for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, t, peer, group, tag) for t in tensors]):
                w.wait()                 # stream-level wait only; the host does not block
            return
        for t in tensors:
            w = dist.isend(t, dst=peer, group=group, tag=tag)
            if self.cuda:
                w.wait()
            else:
                self.pending.append(_Hold(w, t))

    def _recv(self, node: TrainingDAGNode) -> None:
        a = self.a
        m = node.node_meta
        peer = a.layout.peer_rank(m["peer_pp_rank"])
        group, tag = self._channel(node)
        consumer = self.dag.nodes[m["to_uid"]]
        if consumer.compute_subkind == "FWD":
            metas = a.buckets[consumer.node_meta["bucket_key"]].input_meta
        else:
            metas = self.shape_ref[consumer.node_meta["fwd_uid"]]
        bufs, works = [], []
        if self.cuda and len(metas) > 1:
            bufs = [torch.empty(shape, dtype=dtype, device=a.device) for shape, dtype in metas]
            for w in dist.batch_isend_irecv([dist.P2POp(dist.irecv, b, peer, group, tag) for b in bufs]):
                w.wait()
            metas = []
        for shape, dtype in metas:
            buf = torch.empty(shape, dtype=dtype, device=a.device)
            w = dist.irecv(buf, src=peer, group=group, tag=tag)
            if self.cuda:
                w.wait()
            else:
                works.append(w)
            bufs.append(buf)
        self.outs[node.uid] = tuple(bufs)
        self._works[node.uid] = works

    def _storage_of(self, node: TrainingDAGNode) -> Optional[ParamStorage]:
        b = self.a.buckets.get(node.node_meta.get("bucket_key"))
        return None if b is None else b.storage

    def _all_reduce(self, node: TrainingDAGNode) -> None:
        if node.node_meta.get("noop"):
            return
        st = self._storage_of(node)
        if st is None or st.mode != "allreduce":
            return
        a = self.a
        if a.fused is not None and a.fused.supports(st):
            a.fused.reduce(st, True, 1.0 / (a.num_microbatches * a.layout.dp_degree))
        else:
            st.all_reduce_grads(per_tensor=(a.baseline == "nccl"))

    def _reduce_scatter(self, node: TrainingDAGNode) -> None:
        st = self._storage_of(node)
        if st is None or st.mode not in ("zero2", "zero3"):
            return
        if not st.release_grads():
            if node.node_meta.get("zero_free_full_params_after"):
                self._free_params(st, node)
            return
        a = self.a
        if a.fused is not None and a.fused.supports(st):
            a.fused.reduce(st, bool(node.node_meta.get("last_sync")), 1.0 / (a.num_microbatches * a.layout.dp_degree))
            if node.node_meta.get("zero_free_full_params_after"):
                self._free_params(st, node)
            return
        st.reduce_scatter_grads()
        if st.mode == "zero3":
            st.free_grads(self.a.streams.get(node.stream) if self.cuda else None)
        else:
            st.flat_grads.zero_()
        if node.node_meta.get("zero_free_full_params_after"):
            st.free_params(self.a.streams.get(node.stream) if self.cuda else None)

    def _all_gather(self, node: TrainingDAGNode) -> None:
        st = self._storage_of(node)
        if st is None or st.mode != "zero3":
            return
        a = self.a
        if a.fused is not None and a.fused.supports(st):
            consumer = self.dag.nodes.get(node.node_meta.get("compute_uid"))
            fwd = consumer is not None and consumer.node_kind == COMPUTE and consumer.compute_subkind == "FWD" \
                and not a.activation_checkpointing
            a.fused.gather(st, fuse_first=fwd)
        else:
            st.all_gather_params()

    def _free_params(self, st: ParamStorage, node: TrainingDAGNode) -> None:
        if self.a.fused is not None and self.a.fused.supports(st) and st.param_users <= 1:
            self.a.fused.release(st)
        st.free_params(self.a.streams.get(node.stream) if self.cuda else None)

    def _all_to_all(self, node: TrainingDAGNode) -> None:
        from ..parallel.expert import exchange_tokens
        m = node.node_meta
        src = self.dag.data_preds(node.uid)[0]
        vals = list(self.outs[src])
        self._wait_work(src)
        ef = self.a.ep_fused
        if ef is not None and ef.supports(node):
            res = ef.exchange(node, vals)
        else:
            res = exchange_tokens(self, node, vals)
        self.outs[node.uid] = res
        self._drop_exchanged(src, node, vals, res)

    def _update(self, node: TrainingDAGNode) -> None:
        a = self.a
        scale = 1.0 / (a.num_microbatches * a.layout.dp_degree)
        if a.debug_keep_grads:
            a.last_grads = {}
        for b in a.buckets.values():
            st = b.storage
            if st is None or st.numel == 0:
                continue
            if st.replica_group is not None and st.flat_grads is not None:
                dist.all_reduce(st.flat_grads, group=st.replica_group)
            if a.debug_keep_grads:
                a.last_grads.update(st.snapshot_grads(scale))
            if getattr(st, "fused_stepped", False):
                st.fused_stepped = False
                continue
            st.step(scale)


class _Hold:
    """Keeps a tensor alive until its asynchronous send has completed."""

    def __init__(self, work, tensor) -> None:
        self.work, self.tensor = work, tensor

    def wait(self) -> None:
        self.work.wait()
        self.tensor = None
