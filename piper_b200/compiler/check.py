"""Static checks of the per-rank plans before anything is launched.

The executor issues every node of a rank in one fixed dispatch order onto FIFO streams and turns every edge that
crosses streams into an event wait.  Three things can still go wrong in a schedule, and all of them would show up
as a hang or as silently swapped pipeline messages on the GPUs; ``check_plans`` finds them on the host instead:

1. *order*: the dispatch order of a rank must place the source of every data / temporal edge before its
   destination (otherwise an event would be waited for before it is recorded);
2. *channel FIFO*: messages of one pipeline channel are matched by position, so the k-th send a sender issues on a
   channel must be the partner of the k-th receive its peer issues on that channel;
3. *deadlock*: a send and its receive complete together.  With each such pair merged into one node, the union of
   all ranks' edges, per-stream issue order and merged pairs must be acyclic; a cycle means some stream waits
   (through events and the rendezvous of a message) on work queued behind itself.

The reference has no such checker; it relies on assertions inside its ZeRO planner and on cycle checks for
``order`` directives (``src/directives.py:1450-1474``), and leaves cross-rank consistency to the NCCL watchdog.
"""
from __future__ import annotations

from typing import Optional

from .dag import RECV, SEND, TrainingDAG
from .ordering import serial_topological_order


class PlanError(RuntimeError):
    """A per-rank plan that would hang or mis-deliver messages."""


def _stream_key(dag: TrainingDAG, uid: str):
    n = dag.nodes[uid]
    if n.node_kind in (SEND, RECV):
        return ("channel", n.node_meta.get("channel_base") or n.node_meta.get("channel") or uid)
    return ("stream", n.stream)


def check_plans(per_device: list, orders: Optional[list] = None) -> dict:
    """Validate the plans of all pipeline ranks together; returns counters, raises ``PlanError`` on a defect.

    ``per_device[r]`` is the DAG of pipeline rank ``r`` (data-parallel replicas share it); ``orders[r]`` its
    dispatch order (computed the way the actor does when omitted).
    """
    if orders is None:
        orders = [serial_topological_order(d) for d in per_device]
    pos = []
    for r, (dag, order) in enumerate(zip(per_device, orders)):
        if sorted(order) != sorted(dag.nodes):
            raise PlanError(f"rank {r}: dispatch order does not cover the DAG exactly once")
        where = {uid: i for i, uid in enumerate(order)}
        pos.append(where)
        for e in dag.edges:
            if where[e.src_uid] >= where[e.dst_uid]:
                raise PlanError(f"rank {r}: {e.dst_uid} is dispatched before its {e.dep_kind} predecessor {e.src_uid}")

    # ---- channel FIFO: partner of the k-th send == k-th receive of that channel on the peer
    owner = {}
    for r, dag in enumerate(per_device):
        for uid in dag.nodes:
            owner[uid] = r
    sends: dict = {}
    recvs: dict = {}
    for r, (dag, order) in enumerate(zip(per_device, orders)):
        for uid in order:
            n = dag.nodes[uid]
            if n.node_kind == SEND:
                sends.setdefault(_stream_key(dag, uid), []).append(uid)
            elif n.node_kind == RECV:
                recvs.setdefault(_stream_key(dag, uid), []).append(uid)
    pairs = []
    for key in sorted(set(sends) | set(recvs), key=repr):
        s_list, r_list = sends.get(key, []), recvs.get(key, [])
        if len(s_list) != len(r_list):
            raise PlanError(f"channel {key[1]}: {len(s_list)} sends but {len(r_list)} receives")
        for k, (s_uid, r_uid) in enumerate(zip(s_list, r_list)):
            partner = per_device[owner[s_uid]].nodes[s_uid].node_meta.get("pair_uid")
            if partner is not None and partner != r_uid:
                raise PlanError(f"channel {key[1]}: message {k} is sent by {s_uid} for {partner} "
                                f"but the peer's receive number {k} is {r_uid}")
            pairs.append((s_uid, r_uid))

    # ---- deadlock: merge each send with its receive, add issue order per stream, look for a cycle
    rep = {}
    for s_uid, r_uid in pairs:
        rep[(owner[r_uid], r_uid)] = (owner[s_uid], s_uid)

    def node(r, uid):
        return rep.get((r, uid), (r, uid))

    succ: dict = {}
    indeg: dict = {}

    def add_edge(a, b):
        if a == b:
            return
        if b not in succ.setdefault(a, set()):
            succ[a].add(b)
            indeg[b] = indeg.get(b, 0) + 1
        indeg.setdefault(a, indeg.get(a, 0))

    for r, (dag, order) in enumerate(zip(per_device, orders)):
        for uid in order:
            indeg.setdefault(node(r, uid), 0)
        for e in dag.edges:
            sk, dk = dag.nodes[e.src_uid].node_kind, dag.nodes[e.dst_uid].node_kind
            if e.dep_kind == "temporal" and sk in (SEND, RECV) and dk in (SEND, RECV):
                continue          # ordered by host issue only, never waited for on the device
            add_edge(node(r, e.src_uid), node(r, e.dst_uid))
        last: dict = {}
        for uid in order:
            key = _stream_key(dag, uid)
            if key in last:
                add_edge(node(r, last[key]), node(r, uid))
            last[key] = uid
    ready = sorted(n for n, d in indeg.items() if d == 0)
    done = 0
    while ready:
        cur = ready.pop()
        done += 1
        for nxt in sorted(succ.get(cur, ())):
            indeg[nxt] -= 1
            if indeg[nxt] == 0:
                ready.append(nxt)
    if done != len(indeg):
        stuck = sorted(f"rank{r}:{uid}" for (r, uid), d in indeg.items() if d > 0)
        raise PlanError("the plans can deadlock: these nodes wait on one another through events, stream order and "
                        f"message rendezvous: {', '.join(stuck[:12])}{' ...' if len(stuck) > 12 else ''}")
    return {"ranks": len(per_device), "nodes": sum(len(d.nodes) for d in per_device), "messages": len(pairs)}
