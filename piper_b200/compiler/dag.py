"""Training-DAG IR.

A ``TrainingDAG`` holds one node per schedulable task of a training step
(forward / backward compute of an annotated model segment, the optimizer
update, and the communication tasks that schedule directives insert) and
``data`` / ``temporal`` edges between them.  The node and edge records have
the same fields as the reference IR (``src/dag.py:23-66``) so that schedules,
tests and visualisations written against it keep working; the container
differs: edges are indexed per endpoint (the reference scans a flat list in
most helpers, ``src/zero.py:45-55``, ``src/dag.py:252-260``), parallel edges
between the same pair are reference-counted so removing one keeps the
adjacency of the other, and every traversal is deterministic so that all
ranks, which each run the compiler, derive identical plans.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterable, Iterator, Optional

COMPUTE = "COMPUTE"
UPD = "UPD"
SEND = "SEND_COMM"
RECV = "RECV_COMM"
REDUCE = "REDUCE_COMM"
ALL_GATHER = "ALL_GATHER_COMM"
REDUCE_SCATTER = "REDUCE_SCATTER_COMM"
A2A = "A2A_COMM"
ORDER_DUMMY = "ORDER_DUMMY"
DEFAULT_STREAM = "default_stream"
STASH_EDGE = "__activations__"   # tensor_name of the forward -> own backward edge


@dataclass(frozen=True)
class TrainingDAGEdge:
    src_uid: str
    dst_uid: str
    dep_kind: str  # "data" | "temporal"
    tensor_name: Optional[str] = None

    @property
    def key(self) -> tuple:
        return (self.src_uid, self.dst_uid, self.dep_kind, self.tensor_name)


@dataclass
class TrainingDAGNode:
    uid: str
    node_kind: str
    compute_subkind: Optional[str]  # FWD | BWD | BWD_I | BWD_W for COMPUTE nodes
    tag: dict
    device: Optional[list]
    stream: str
    node_meta: dict = field(default_factory=dict)

    def clone(self, **changes) -> "TrainingDAGNode":
        n = TrainingDAGNode(
            uid=self.uid,
            node_kind=self.node_kind,
            compute_subkind=self.compute_subkind,
            tag=dict(self.tag),
            device=None if self.device is None else list(self.device),
            stream=self.stream,
            node_meta=dict(self.node_meta),
        )
        for k, v in changes.items():
            setattr(n, k, v)
        return n

    @property
    def device_key(self) -> Optional[tuple]:
        return None if self.device is None else tuple(sorted(int(d) for d in self.device))


class TrainingDAG:
    """Directed multigraph with per-endpoint edge indices."""

    def __init__(self) -> None:
        self.nodes: dict[str, TrainingDAGNode] = {}
        self._edges: dict[tuple, TrainingDAGEdge] = {}
        self._out: dict[str, dict[tuple, TrainingDAGEdge]] = {}
        self._in: dict[str, dict[tuple, TrainingDAGEdge]] = {}
        self._pair_count: dict[tuple[str, str], int] = {}
        self.succs: dict[str, set[str]] = {}
        self.preds: dict[str, set[str]] = {}

    # ------------------------------------------------------------ mutation
    def add_node(self, node: TrainingDAGNode) -> TrainingDAGNode:
        if node.uid in self.nodes:
            raise ValueError(f"Duplicate node uid: {node.uid}")
        self.nodes[node.uid] = node
        self._out[node.uid] = {}
        self._in[node.uid] = {}
        self.succs[node.uid] = set()
        self.preds[node.uid] = set()
        return node

    def add_edge(self, edge: TrainingDAGEdge) -> None:
        if edge.src_uid not in self.nodes or edge.dst_uid not in self.nodes:
            raise ValueError(f"Edge references unknown node: {edge}")
        k = edge.key
        if k in self._edges:
            return
        self._edges[k] = edge
        self._out[edge.src_uid][k] = edge
        self._in[edge.dst_uid][k] = edge
        pair = (edge.src_uid, edge.dst_uid)
        self._pair_count[pair] = self._pair_count.get(pair, 0) + 1
        self.succs[edge.src_uid].add(edge.dst_uid)
        self.preds[edge.dst_uid].add(edge.src_uid)

    def connect(self, src: str, dst: str, kind: str = "data", tensor_name: Optional[str] = None) -> None:
        self.add_edge(TrainingDAGEdge(src, dst, kind, tensor_name))

    def remove_edge(self, edge: TrainingDAGEdge) -> None:
        k = edge.key
        if k not in self._edges:
            return
        del self._edges[k]
        del self._out[edge.src_uid][k]
        del self._in[edge.dst_uid][k]
        pair = (edge.src_uid, edge.dst_uid)
        self._pair_count[pair] -= 1
        if self._pair_count[pair] == 0:
            del self._pair_count[pair]
            self.succs[edge.src_uid].discard(edge.dst_uid)
            self.preds[edge.dst_uid].discard(edge.src_uid)

    def remove_node(self, uid: str) -> None:
        if uid not in self.nodes:
            return
        for e in list(self._out[uid].values()) + list(self._in[uid].values()):
            self.remove_edge(e)
        del self.nodes[uid], self._out[uid], self._in[uid], self.succs[uid], self.preds[uid]

    def bypass_node(self, uid: str, kinds: tuple = ("data",)) -> None:
        """Remove ``uid`` and reconnect each predecessor to each successor (for the given edge kinds)."""
        ins = [e for e in self.in_edges(uid) if e.dep_kind in kinds]
        outs = [e for e in self.out_edges(uid) if e.dep_kind in kinds]
        for ie in ins:
            for oe in outs:
                self.connect(ie.src_uid, oe.dst_uid, oe.dep_kind,
                             oe.tensor_name if oe.tensor_name is not None else ie.tensor_name)
        self.remove_node(uid)

    # ------------------------------------------------------------- queries
    @property
    def edges(self) -> list[TrainingDAGEdge]:
        return list(self._edges.values())

    @property
    def edge_keys(self) -> set[tuple]:
        return set(self._edges.keys())

    def out_edges(self, uid: str, kind: Optional[str] = None) -> list[TrainingDAGEdge]:
        es = self._out.get(uid, {}).values()
        return [e for e in es if kind is None or e.dep_kind == kind]

    def in_edges(self, uid: str, kind: Optional[str] = None) -> list[TrainingDAGEdge]:
        es = self._in.get(uid, {}).values()
        return [e for e in es if kind is None or e.dep_kind == kind]

    def has_edge(self, src: str, dst: str, kind: Optional[str] = None) -> bool:
        return any(e.dst_uid == dst for e in self.out_edges(src, kind))

    def data_preds(self, uid: str) -> list[str]:
        return [e.src_uid for e in self.in_edges(uid, "data")]

    def data_succs(self, uid: str) -> list[str]:
        return [e.dst_uid for e in self.out_edges(uid, "data")]

    def __len__(self) -> int:
        return len(self.nodes)

    def __iter__(self) -> Iterator[TrainingDAGNode]:
        return iter(self.nodes.values())

    def select(self, pred) -> list[TrainingDAGNode]:
        return [n for n in self.nodes.values() if pred(n)]

    def copy_subgraph(self, uids: Iterable[str]) -> "TrainingDAG":
        keep = set(uids)
        sub = TrainingDAG()
        for uid, n in self.nodes.items():
            if uid in keep:
                sub.add_node(n.clone())
        for e in self._edges.values():
            if e.src_uid in keep and e.dst_uid in keep:
                sub.add_edge(e)
        return sub

    # ----------------------------------------------------------- traversal
    def topological_order(self) -> list[str]:
        """Level-synchronous Kahn order; ties inside a level break by uid."""
        indeg = {uid: len(self._in[uid]) for uid in self.nodes}
        frontier = sorted(uid for uid, d in indeg.items() if d == 0)
        order: list[str] = []
        while frontier:
            nxt: list[str] = []
            for u in frontier:
                order.append(u)
                for e in self._out[u].values():
                    indeg[e.dst_uid] -= 1
                    if indeg[e.dst_uid] == 0:
                        nxt.append(e.dst_uid)
            nxt.sort()
            frontier = nxt
        if len(order) != len(self.nodes):
            stuck = sorted(uid for uid, d in indeg.items() if d > 0)
            raise ValueError(f"TrainingDAG topological sort failed: cycle through {stuck[:8]}")
        return order

    def topological_levels(self, order: Optional[list[str]] = None) -> dict[str, int]:
        levels: dict[str, int] = {}
        for uid in order or self.topological_order():
            ps = self.preds[uid]
            levels[uid] = 1 + max(levels[p] for p in ps) if ps else 0
        return levels

    def has_path(self, src: str, dst: str) -> bool:
        if src == dst:
            return True
        seen = {src}
        stack = [src]
        while stack:
            for v in self.succs[stack.pop()]:
                if v == dst:
                    return True
                if v not in seen:
                    seen.add(v)
                    stack.append(v)
        return False

    def descendants(self, uid: str) -> set[str]:
        seen: set[str] = set()
        stack = [uid]
        while stack:
            for v in self.succs[stack.pop()]:
                if v not in seen:
                    seen.add(v)
                    stack.append(v)
        return seen

    def ancestors(self, uid: str) -> set[str]:
        seen: set[str] = set()
        stack = [uid]
        while stack:
            for v in self.preds[stack.pop()]:
                if v not in seen:
                    seen.add(v)
                    stack.append(v)
        return seen


def with_pass_tag(tag: dict, pass_value: Optional[str]) -> dict:
    t = dict(tag)
    t["PASS"] = pass_value
    return t


def is_compute(node: TrainingDAGNode, *subkinds: str) -> bool:
    return node.node_kind == COMPUTE and (not subkinds or node.compute_subkind in subkinds)


def build_training_dag(segments: list) -> TrainingDAG:
    """One FWD node per annotated segment, mirrored BWD nodes, and the update node.

    Forward nodes ``s{stage}.seg{i}`` are chained by data edges in segment order;
    every forward edge u->v has a backward edge v.bwd->u.bwd; the last forward
    feeds the first backward (which computes the loss); ``upd.0`` waits on every
    backward through temporal edges (``src/dag.py:101-241`` has the same shape).
    """
    dag = TrainingDAG()
    fwd_uids: list[str] = []
    for seg in segments:
        uid = f"s{seg.stage_id}.seg{seg.segment_id}"
        gm = seg.gm
        in_names = [n.name for n in gm.graph.nodes if n.op == "placeholder"]
        dag.add_node(TrainingDAGNode(
            uid=uid, node_kind=COMPUTE, compute_subkind="FWD", tag=with_pass_tag(seg.tag, "F"),
            device=None, stream=DEFAULT_STREAM,
            node_meta={
                "bucket_key": uid,
                "stage_id": seg.stage_id,
                "segment_id": seg.segment_id,
                "gm": gm,
                "input_idxs": list(seg.input_idxs),
                "param_idxs": list(seg.param_idxs),
                "graphargs": list(seg.graphargs),
                "param_fqns": list(getattr(seg, "param_fqns", [])),
                "input_names": in_names,
                "output_names": list(getattr(seg, "output_names", [])),
                "a2a_boundary_after": seg.a2a_boundary_after,
                "a2a_boundary_before": getattr(seg, "a2a_boundary_before", None),
            },
        ))
        if fwd_uids:
            dag.connect(fwd_uids[-1], uid, "data")
        fwd_uids.append(uid)

    for f in fwd_uids:
        fn = dag.nodes[f]
        dag.add_node(TrainingDAGNode(
            uid=f"{f}.bwd", node_kind=COMPUTE, compute_subkind="BWD", tag=with_pass_tag(fn.tag, "B"),
            device=None, stream=DEFAULT_STREAM,
            node_meta={"fwd_uid": f, "bucket_key": fn.node_meta["bucket_key"], "compute_loss": False},
        ))
    for a, b in zip(fwd_uids, fwd_uids[1:]):
        dag.connect(f"{b}.bwd", f"{a}.bwd", "data")
    # a backward consumes the activations its forward stashed: a real dependency that also keeps the forward
    # and backward halves of a pipeline rank in one connected component when no order directive links them
    for f in fwd_uids:
        dag.connect(f, f"{f}.bwd", "data", STASH_EDGE)
    if fwd_uids:
        last = max(fwd_uids, key=lambda u: (dag.nodes[u].node_meta["stage_id"], dag.nodes[u].node_meta["segment_id"]))
        dag.connect(last, f"{last}.bwd", "data")
        dag.nodes[f"{last}.bwd"].node_meta["compute_loss"] = True

    dag.add_node(TrainingDAGNode(uid="upd.0", node_kind=UPD, compute_subkind=None, tag={"PASS": None},
                                 device=None, stream=DEFAULT_STREAM, node_meta={}))
    for f in fwd_uids:
        dag.connect(f"{f}.bwd", "upd.0", "temporal")
    return dag


# Function-style aliases with the reference's names, for code written against it.
def _topological_order(dag: TrainingDAG) -> list[str]:
    return dag.topological_order()


def _topological_levels(dag: TrainingDAG) -> dict[str, int]:
    return dag.topological_levels()


def _has_path(dag: TrainingDAG, src: str, dst: str) -> bool:
    return dag.has_path(src, dst)
