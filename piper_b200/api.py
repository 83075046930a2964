"""User-facing API: ``annotate``, the ``piper`` Dynamo backend, and the DAG compile pipeline.

``annotate(tag)`` stamps every op traced inside the scope with the stack of
enclosing scopes (name, auto-assigned index per name, unique id) through
``torch.fx.traceback.annotate``, so TorchDynamo copies it into
``node.meta["custom"]["piper_annotations"]`` (same mechanism and metadata key
as ``src/piper.py:51-80``).  The backend registered as ``"piper"`` turns the
captured graph into per-device training DAGs and stores them in
``piper_metadata``; the callable it returns only runs the captured graph
locally.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Iterator, Optional

import torch.fx as fx
from torch._dynamo.backends.registry import register_backend

from .compiler.dag import TrainingDAG, build_training_dag
from .compiler.decompose import split_by_device_set
from .compiler.directives import apply_schedule_directives, validate_schedule_tags_exist
from .compiler.fxsplit import PIPER_ANNOTATIONS_META_KEY, split_gm_by_annotations
from .compiler.ordering import resolve_total_order_per_stream
from .compiler.zero import add_inter_chain_temporal_edges, prune_zero_lifetimes
from .state import LOG_LEVEL, create_logger, piper_metadata

logger = create_logger("piper_backend", LOG_LEVEL)

_STACK: list[dict] = []
_COUNTS: dict[str, int] = {}
_NEXT_UID = 0


def _reset_annotation_state() -> None:
    global _NEXT_UID
    _STACK.clear()
    _COUNTS.clear()
    _NEXT_UID = 0


@contextmanager
def annotate(name: str) -> Iterator[dict]:
    """Mark the enclosed model code as schedule region ``name``; indices count up per name in trace order."""
    if not isinstance(name, str) or not name:
        raise ValueError(f"piper.annotate requires a non-empty string tag name, got {name!r}")
    global _NEXT_UID
    index = _COUNTS.get(name, 0)
    _COUNTS[name] = index + 1
    entry = {"name": name, "index": int(index), "uid": int(_NEXT_UID)}
    _NEXT_UID += 1
    _STACK.append(entry)
    try:
        with fx.traceback.annotate({PIPER_ANNOTATIONS_META_KEY: tuple(dict(e) for e in _STACK),
                                    "name": name, "index": int(index)}):
            yield entry
    finally:
        top = _STACK.pop()
        if top is not entry:
            raise RuntimeError("piper.annotate stack corrupted during tracing")


def compile_training_dags(gm: fx.GraphModule, directives: Optional[list], *, visualize: bool = False,
                          artifact_dir: str = "out") -> tuple[TrainingDAG, list[TrainingDAG], list]:
    """graph -> segments -> global DAG -> directives -> per-device DAGs (pruned, totally ordered)."""
    _gm, segments = split_gm_by_annotations(gm)
    if not segments:
        raise ValueError("No Piper annotations found in the traced graph. Wrap model compute with "
                         "piper.annotate(...) before compiling with Piper.")
    dag = build_training_dag(segments)
    validate_schedule_tags_exist(dag, directives)
    apply_schedule_directives(dag, directives)
    per_device = split_by_device_set(dag) if any(n.device is not None for n in dag.nodes.values()) else [dag]
    for i, sub in enumerate(per_device):
        chains = prune_zero_lifetimes(sub)
        resolve_total_order_per_stream(sub)
        add_inter_chain_temporal_edges(sub, chains)
        if visualize:
            from .compiler import viz
            viz.print_training_dag_order(sub, label=f"pp{i}", rank=i, out_dir=artifact_dir)
            viz.render_training_dag(sub, output_path=f"{artifact_dir}/training_dag_pp{i}")
    return dag, per_device, segments


@register_backend
def piper(gm, example_inputs, **kwargs):
    """TorchDynamo backend: compile the captured graph into per-device training DAGs."""
    del example_inputs, kwargs
    dag, per_device, segments = compile_training_dags(
        gm, getattr(piper_metadata, "schedule_directives", None),
        visualize=bool(getattr(piper_metadata, "visualize_dag", False)),
        artifact_dir=getattr(piper_metadata, "artifact_dir", "out"))
    piper_metadata.training_dag = dag
    piper_metadata.per_pp_training_dags = per_device
    piper_metadata.segments = segments
    logger.debug("built TrainingDAG with %d nodes and %d edges, split into %d per-device DAG(s)",
                 len(dag.nodes), len(dag.edges), len(per_device))

    def run_locally(*args, _gm=gm):
        import torch
        if not any(isinstance(a, torch.Tensor) and a.is_meta for a in args):
            logger.warning("piper compiled callback invoked directly; running local graph execution")
        return _gm(*args)

    return run_locally
