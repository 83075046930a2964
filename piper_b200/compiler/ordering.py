"""Total order of a per-device training DAG.

Three steps, behaviourally the same as the reference (``src/ordering.py``):

1. *Default-stream serialisation*: while two default-stream compute nodes
   share a topological level, chain them with temporal edges, the node with
   more transitive successors first (ties by uid).
2. *Side-stream chaining*: nodes of every other logical stream are ordered by
   the position of the default-stream node they touch and chained with
   temporal edges (an ordering that would close a cycle is an error).
3. *Dispatch order*: sort by ``(level, priority, topological index)`` with
   priority SEND < ALL_GATHER/A2A < REDUCE/REDUCE_SCATTER < compute/UPD/dummy
   < RECV.

Step 1 here keeps the transitive-successor counts cached and recomputes
levels once per inserted chain, not once per edge.
"""
from __future__ import annotations

from typing import Optional

from .dag import (A2A, ALL_GATHER, COMPUTE, DEFAULT_STREAM, RECV, REDUCE, REDUCE_SCATTER, SEND, TrainingDAG)

_PRIORITY = {SEND: 0, ALL_GATHER: 1, A2A: 1, REDUCE: 2, REDUCE_SCATTER: 2, RECV: 4}


def serial_topological_order(dag: TrainingDAG, levels: Optional[dict[str, int]] = None) -> list[str]:
    base = dag.topological_order()
    if levels is None:
        levels = dag.topological_levels(base)
    idx = {u: i for i, u in enumerate(base)}
    return sorted(dag.nodes, key=lambda u: (levels[u], _PRIORITY.get(dag.nodes[u].node_kind, 3), idx[u]))


def resolve_default_stream_order(dag: TrainingDAG) -> None:
    uids = [u for u, n in dag.nodes.items() if n.stream == DEFAULT_STREAM and n.node_kind == COMPUTE]
    if len(uids) < 2:
        return
    downstream = {u: len(dag.descendants(u)) for u in uids}
    while True:
        levels = dag.topological_levels()
        by_level: dict[int, list[str]] = {}
        for u in uids:
            by_level.setdefault(levels[u], []).append(u)
        clash = next((lv for lv in sorted(by_level) if len(by_level[lv]) > 1), None)
        if clash is None:
            return
        chain = sorted(by_level[clash], key=lambda u: (-downstream[u], u))
        for a, b in zip(chain, chain[1:]):
            dag.connect(a, b, "temporal")
        # successor counts of chain members and of their ancestors changed
        touched = set(chain)
        for u in chain:
            touched |= dag.ancestors(u)
        for u in uids:
            if u in touched:
                downstream[u] = len(dag.descendants(u))


def resolve_total_order_per_stream(dag: TrainingDAG) -> None:
    resolve_default_stream_order(dag)
    topo = dag.topological_order()
    idx = {u: i for i, u in enumerate(topo)}
    levels = dag.topological_levels(topo)
    default_uids = [u for u in topo if dag.nodes[u].stream == DEFAULT_STREAM]
    streams = sorted({n.stream for n in dag.nodes.values() if n.stream != DEFAULT_STREAM})
    if not default_uids or not streams:
        return
    for stream in streams:
        by_anchor: dict[str, list[str]] = {}
        for uid, node in dag.nodes.items():
            if node.stream != stream:
                continue
            anchors = [e.src_uid for e in dag.in_edges(uid) if dag.nodes[e.src_uid].stream == DEFAULT_STREAM]
            anchors += [e.dst_uid for e in dag.out_edges(uid) if dag.nodes[e.dst_uid].stream == DEFAULT_STREAM]
            if not anchors:
                continue
            anchor = min(anchors, key=lambda a: (levels[a], idx[a]))
            by_anchor.setdefault(anchor, []).append(uid)
        cur = None
        for d in default_uids:
            for nxt in sorted(set(by_anchor.get(d, [])), key=lambda u: (levels[u], idx[u])):
                if cur is not None and cur != nxt:
                    if dag.has_path(nxt, cur):
                        raise ValueError(
                            f"resolve_total_order_per_stream would create a cycle while ordering "
                            f"stream={stream}: {cur} -> {nxt}")
                    if not dag.has_path(cur, nxt):
                        dag.connect(cur, nxt, "temporal")
                cur = nxt


# reference-compatible names
_serial_topological_order = serial_topological_order
_resolve_default_stream_order = resolve_default_stream_order
