"""``src.tasks`` of the reference: node kinds the executor dispatches on (``src/tasks.py:8-51``).

This runtime dispatches directly on ``(node_kind, compute_subkind)`` of the DAG node; ``task_type`` gives the
reference's task name for a node, for tools that label traces with it.
"""
from piper_b200.compiler.dag import (ALL_GATHER, COMPUTE, ORDER_DUMMY, RECV, REDUCE, REDUCE_SCATTER, SEND,  # noqa: F401
                                     UPD, TrainingDAGNode)

_BY_KIND = {SEND: "SEND", RECV: "RECV", REDUCE: "ALL_REDUCE", ALL_GATHER: "ALL_GATHER",
            REDUCE_SCATTER: "REDUCE_SCATTER", UPD: "UPDATE", ORDER_DUMMY: "DUMMY", "A2A_COMM": "ALL_TO_ALL"}
_BY_SUBKIND = {"FWD": "FORWARD", "BWD": "BACKWARD", "BWD_I": "BACKWARD_INPUT", "BWD_W": "BACKWARD_WEIGHT"}


def task_type(node: TrainingDAGNode) -> str:
    if node.node_kind == COMPUTE:
        return _BY_SUBKIND.get(node.compute_subkind, "FORWARD")
    return _BY_KIND.get(node.node_kind, node.node_kind)
