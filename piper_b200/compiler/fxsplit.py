"""Splitting a traced ``GraphModule`` into annotated segments.

Every compute node of the Dynamo graph carries the stack of enclosing
``piper.annotate`` scopes in ``node.meta["custom"]["piper_annotations"]``.
Maximal runs of consecutive nodes with the same stack (uid included, so two
consecutive ``annotate("PP")`` scopes are two segments) become
``AnnotationSegment`` s, each with its own ``GraphModule`` whose placeholders
are, in this order: the runtime inputs (model inputs for the first segment,
the live values crossing in from earlier segments otherwise, named
``_xseg_<name>``) and then the parameters / buffers it reads.  Values that
are needed further downstream are forwarded through every segment in
between, so the segments form a chain (``src/fx.py:506-702`` has the same
contract).

Two things are decided differently from the reference:

* A placeholder is a *runtime input* when Dynamo's source for it is a plain
  local of the traced function that is not rooted at the module; the
  reference keys on ``"grapharg" in node.meta``, which is true for every
  placeholder while a backend runs, and thereby turns the token input into a
  zero-filled parameter slot (``src/fx.py:399-409``).
* The tensor exchanged at an expert-parallel boundary is chosen by dataflow:
  the floating-point value that the next segment's compute actually
  consumes (and, if present, the integer per-expert row counts next to it),
  never "the first float that is live" (``src/fx.py:486-503`` picks the
  residual stream).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.fx as fx

PIPER_ANNOTATIONS_META_KEY = "piper_annotations"
_NON_COMPUTE = ("placeholder", "get_attr", "output")


@dataclass
class AnnotationSegment:
    segment_id: int
    stage_id: int
    tag: dict
    gm: fx.GraphModule
    input_idxs: list
    param_idxs: list
    graphargs: list
    placeholders: list
    a2a_boundary_after: Optional[dict] = None
    a2a_boundary_before: Optional[dict] = None
    param_fqns: list = field(default_factory=list)     # per placeholder position; None for runtime inputs
    output_names: list = field(default_factory=list)


def example_value(node: fx.Node) -> Any:
    return node.meta.get("example_value", node.meta.get("val"))


def annotation_stack(node: fx.Node) -> tuple:
    custom = node.meta.get("custom")
    if not isinstance(custom, dict) or PIPER_ANNOTATIONS_META_KEY not in custom:
        return ()
    raw = custom[PIPER_ANNOTATIONS_META_KEY]
    if not isinstance(raw, (list, tuple)) or not raw:
        raise ValueError("Piper annotation metadata must be a non-empty list/tuple of "
                         f"{{'name': str, 'index': int, 'uid': int}} entries. Node {node.name!r} has {raw!r}.")
    out = []
    for a in raw:
        if not isinstance(a, dict) or set(a) - {"name", "index", "uid"}:
            raise ValueError(f"Piper annotation entries may only contain 'name', 'index', and 'uid'. "
                             f"Node {node.name!r} has {a!r}.")
        name, index, uid = a.get("name"), a.get("index"), a.get("uid")
        if not isinstance(name, str) or not name or not isinstance(index, int) or not isinstance(uid, int):
            raise ValueError(f"malformed Piper annotation on node {node.name!r}: {a!r}")
        out.append((name, int(index), int(uid)))
    return tuple(out)


def _tag(stack: tuple) -> dict:
    return {name: index for name, index, _uid in stack}


_SRC_PART = re.compile(r"\._(modules|parameters|buffers)\['([^']+)'\]|\.([A-Za-z_][A-Za-z_0-9]*)")


def source_fqn(node: fx.Node) -> Optional[str]:
    """Module-qualified name (``layers.0.attention.wq.weight``) of a parameter/buffer placeholder.

    Derived from Dynamo's source expression, e.g.
    ``L['self']._modules['layers']._modules['0']._parameters['weight']``; falls back to decoding the
    placeholder name (``l_self_modules_layers_modules_0_parameters_weight_``).
    """
    if node.meta.get("piper_fqn"):
        return node.meta["piper_fqn"]
    src = getattr(node, "_dynamo_source", None)
    name = getattr(src, "name", None) if src is not None else None
    if callable(name):
        name = name()
    if isinstance(name, str) and ("_parameters[" in name or "_buffers[" in name or "_modules[" in name):
        parts = [m.group(2) or m.group(3) for m in _SRC_PART.finditer(name[name.index("]") + 1:])]
        if parts:
            return ".".join(parts)
    nm = node.name
    if nm.startswith("l_") and ("_parameters_" in nm or "_buffers_" in nm):
        body = nm.split("_", 2)[2] if nm.count("_") >= 2 else nm
        body = body.strip("_")
        body = re.sub(r"^modules_", "", body)
        body = body.replace("_modules_", ".").replace("_parameters_", ".").replace("_buffers_", ".")
        body = re.sub(r"^parameters_|^buffers_", "", body)
        return body
    return None


def placeholder_is_runtime_input(node: fx.Node) -> bool:
    ex = example_value(node)
    if not isinstance(ex, torch.Tensor) or isinstance(ex, torch.nn.Parameter) or ex.requires_grad:
        return False
    src = getattr(node, "_dynamo_source", None)
    if src is not None:
        name = getattr(src, "name", "")
        if callable(name):
            name = name()
        if isinstance(name, str) and name:
            return not any(k in name for k in ("_parameters[", "_buffers[", "_modules[", "['self']"))
    return "self" not in node.name


def _meta_like(ex: Any, *, requires_grad: bool, as_parameter: bool):
    if isinstance(ex, torch.Tensor):
        t = torch.empty(ex.shape, dtype=ex.dtype, device="meta")
    elif isinstance(ex, (bool, torch.SymBool)):
        t = torch.empty((1,), dtype=torch.bool, device="meta")
    elif isinstance(ex, (int, torch.SymInt)):
        t = torch.empty((1,), dtype=torch.int64, device="meta")
    else:
        t = torch.empty((1,), dtype=torch.float32, device="meta")
    if requires_grad and t.is_floating_point():
        t.requires_grad_(True)
    return torch.nn.Parameter(t, requires_grad=t.requires_grad) if as_parameter else t


def _arg_nodes(x: Any, acc: Optional[list] = None) -> list:
    acc = [] if acc is None else acc
    if isinstance(x, fx.Node):
        acc.append(x)
    elif isinstance(x, (list, tuple)):
        for y in x:
            _arg_nodes(y, acc)
    elif isinstance(x, dict):
        for y in x.values():
            _arg_nodes(y, acc)
    return acc


def _boundary_info(crossing: list, consumers_next: set, produced_prev: set, from_tag: dict, to_tag: dict,
                   ends_in_next: Optional[set] = None) -> dict:
    """Which crossing value an expert-parallel exchange at this boundary moves.

    Preference: a floating-point tensor that the next segment's own compute consumes and that the
    previous segment produced; then one that the next segment consumes; then any float; then index 0.
    ``counts_idx`` is a 1-D integer tensor consumed by the next segment (per-expert row counts), if any.
    """
    def is_float(n):
        ex = example_value(n)
        return isinstance(ex, torch.Tensor) and ex.is_floating_point()

    def pick(pred):
        for i, n in enumerate(crossing):
            if pred(n):
                return i
        return None

    idx = pick(lambda n: is_float(n) and n in consumers_next and n in produced_prev)
    if idx is None:
        idx = pick(lambda n: is_float(n) and n in consumers_next)
    if idx is None:
        idx = pick(lambda n: is_float(n) and n in produced_prev)
    if idx is None:
        idx = pick(is_float)
    if idx is None:
        idx = 0 if crossing else None

    def is_counts(n):
        ex = example_value(n)
        return (isinstance(ex, torch.Tensor) and not ex.is_floating_point() and ex.dtype != torch.bool
                and ex.dim() == 1 and (n in consumers_next or n in produced_prev))

    # the per-expert row counts of an exchange are consumed by the next segment only; an integer vector that
    # merely passes through (and is needed again later) must not be rewritten by the exchange
    cidx = pick(lambda n: is_counts(n) and n in consumers_next and (ends_in_next is None or n in ends_in_next))
    if cidx is None:
        cidx = pick(lambda n: is_counts(n) and n in consumers_next)
    return {"tensor_idx": idx, "counts_idx": cidx, "reshape_input": None, "reshape_output": None,
            "from_tag": from_tag, "to_tag": to_tag}


def split_gm_by_annotations(gm: fx.GraphModule, runtime_input_names: Optional[set] = None
                            ) -> tuple[fx.GraphModule, list[AnnotationSegment]]:
    """Split ``gm`` into annotated segments.  ``runtime_input_names`` overrides the classification of
    placeholders (used when a stage graph, whose inputs are crossing values, is split again into buckets)."""
    nodes = list(gm.graph.nodes)
    compute = [n for n in nodes if n.op not in _NON_COMPUTE]
    stacks = {n: annotation_stack(n) for n in compute}
    if not any(stacks.values()):
        return gm, []
    bare = [n.name for n in compute if not stacks[n]]
    if bare:
        raise ValueError("Found compute nodes without Piper annotations in a graph that uses piper.annotate: "
                         f"{bare[:16]}. Wrap all model compute in piper.annotate(...).")

    seg_of: dict[fx.Node, int] = {}
    seg_stacks: list[tuple] = []
    for n in compute:
        if not seg_stacks or stacks[n] != seg_stacks[-1]:
            seg_stacks.append(stacks[n])
        seg_of[n] = len(seg_stacks) - 1
    n_segs = len(seg_stacks)

    if runtime_input_names is not None:
        runtime_ph = [n for n in nodes if n.op == "placeholder" and n.name in runtime_input_names]
    else:
        runtime_ph = [n for n in nodes if n.op == "placeholder" and placeholder_is_runtime_input(n)]
    param_ph = {n for n in nodes if n.op == "placeholder" and n not in set(runtime_ph)}
    output_node = next((n for n in nodes if n.op == "output"), None)

    # the segment in which each value is defined, and the last segment that reads it
    home = dict(seg_of)
    for n in runtime_ph:
        home[n] = 0
    last_use: dict[fx.Node, int] = {}
    for n, s in home.items():
        uses = [n_segs - 1 if u.op == "output" else seg_of.get(u) for u in n.users]
        uses = [u for u in uses if u is not None]
        last_use[n] = max(uses) if uses else s
    crossing: list[list[fx.Node]] = [[] for _ in range(n_segs)]
    for n in nodes:
        if n in home:
            for t in range(home[n] + 1, last_use[n] + 1):
                crossing[t].append(n)

    segments: list[AnnotationSegment] = []
    for s in range(n_segs):
        g = fx.Graph()
        remap: dict[fx.Node, fx.Node] = {}
        input_idxs, param_idxs, graphargs, fqns = [], [], [], []

        def add_ph(n: fx.Node, name: str, runtime: bool) -> None:
            if n in remap:
                return
            ph = g.placeholder(name)
            ph.type = n.type
            ph.meta.update(n.meta)
            src = getattr(n, "_dynamo_source", None)
            if src is not None:
                try:
                    ph._dynamo_source = src
                except Exception:
                    pass
            remap[n] = ph
            ex = example_value(n)
            rg = bool(getattr(ex, "requires_grad", False))
            pos = len(graphargs)
            if runtime:
                input_idxs.append(pos)
                graphargs.append(_meta_like(ex, requires_grad=rg, as_parameter=False))
                fqns.append(None)
            else:
                param_idxs.append(pos)
                graphargs.append(_meta_like(ex, requires_grad=rg, as_parameter=isinstance(ex, torch.nn.Parameter) or rg))
                fqn = source_fqn(n)
                fqns.append(fqn)
                if fqn:
                    ph.meta["piper_fqn"] = fqn

        if s == 0:
            for n in runtime_ph:
                add_ph(n, n.name, True)
        else:
            for n in crossing[s]:
                add_ph(n, f"_xseg_{n.name}", True)
        body = [n for n in compute if seg_of[n] == s]
        deps: list[fx.Node] = []
        for n in body:
            deps.extend(n.all_input_nodes)
        if output_node is not None and s == n_segs - 1:
            deps.extend(_arg_nodes(output_node.args))
        needed_params = {d for d in deps if d in param_ph}
        needed_attrs = {d for d in deps if d.op == "get_attr"}
        for n in nodes:
            if n in needed_params:
                add_ph(n, n.name, False)
        for n in nodes:
            if n in needed_attrs and n not in remap:
                ga = g.get_attr(n.target)
                ga.type = n.type
                ga.meta.update(n.meta)
                remap[n] = ga
        for n in body:
            missing = [d.name for d in n.all_input_nodes if d not in remap]
            if missing:
                raise ValueError(f"Cannot split annotated graph at segment {s}; node {n.name!r} has unmapped "
                                 f"external dependencies {missing}.")
            remap[n] = g.node_copy(n, lambda x: remap[x])

        before = None
        if s > 0:
            before = segments[-1].a2a_boundary_after
        if s == n_segs - 1:
            out_names: list[str] = []
            if output_node is None:
                g.output(())
            else:
                g.output(fx.map_arg(output_node.args[0], lambda x: remap[x]))
                out_names = [x.name for x in _arg_nodes(output_node.args[0])]
            after = None
        else:
            outs = [remap[n] for n in crossing[s + 1]]
            g.output(tuple(outs) if len(outs) != 1 else outs[0])
            out_names = [n.name for n in crossing[s + 1]]
            nxt_body = [n for n in compute if seg_of[n] == s + 1]
            consumers_next = {d for n in nxt_body for d in n.all_input_nodes}
            ends_next = {n for n in crossing[s + 1] if last_use[n] == s + 1}
            after = _boundary_info(crossing[s + 1], consumers_next, set(body), _tag(seg_stacks[s]),
                                   _tag(seg_stacks[s + 1]), ends_next)
        g.lint()
        seg_gm = fx.GraphModule(gm, g)
        tag = _tag(seg_stacks[s])
        segments.append(AnnotationSegment(
            segment_id=s, stage_id=int(tag.get("PP", s)), tag=tag, gm=seg_gm, input_idxs=input_idxs,
            param_idxs=param_idxs, graphargs=graphargs,
            placeholders=[n for n in seg_gm.graph.nodes if n.op == "placeholder"],
            a2a_boundary_after=after, a2a_boundary_before=before, param_fqns=fqns, output_names=out_names))
    return gm, segments
