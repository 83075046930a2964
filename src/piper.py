"""The reference's ``src.piper`` names, re-exported from ``piper_b200``."""
from piper_b200.api import _reset_annotation_state, annotate, piper  # noqa: F401
from piper_b200.compiler.dag import TrainingDAG, TrainingDAGEdge, TrainingDAGNode, build_training_dag  # noqa: F401
from piper_b200.compiler.decompose import _split_global_training_dag_by_pp_rank  # noqa: F401
from piper_b200.compiler.directives import (  # noqa: F401
    _apply_order_directive, _apply_split_backward_stencil, _apply_split_directive, _bucket_matched_fwd_nodes,
    _parse_order_directive, _validate_schedule_tags_exist, _validate_split_backward_order_stencil,
    apply_schedule_directives)
from piper_b200.compiler.ordering import _serial_topological_order, resolve_total_order_per_stream  # noqa: F401
from piper_b200.engine import piper_exec_dag  # noqa: F401
from piper_b200.state import piper_metadata  # noqa: F401
