"""ZeRO lifetime planning on a per-device DAG.

``replicate(shard_params/shard_grads)`` attaches one ALL_GATHER before and
one REDUCE_SCATTER after every matched compute node.  Most are redundant:
consecutive compute nodes of one parameter bucket that are directly linked
form a *chain* that can share one gathered copy of the parameters and one
full-size gradient buffer.  ``prune_zero_lifetimes`` keeps, per chain, the
all-gather of the head, the parameter free at the tail, the gradient
allocation at the head and the reduce-scatter of the tail (the contract of
``src/zero.py:16-291``).  ``add_inter_chain_temporal_edges`` then orders
successive chains of the same bucket so that a later gather cannot start
before the earlier chain released the buffer, and a later gradient
allocation waits for the earlier reduce-scatter (``src/zero.py:294-369``).

Chains are found with one union-find pass over the edges of each bucket
instead of scanning the whole edge list per node pair.
"""
from __future__ import annotations

from typing import Any

from .dag import ALL_GATHER, COMPUTE, REDUCE, REDUCE_SCATTER, STASH_EDGE, TrainingDAG
from .ordering import serial_topological_order


def _is_compute(dag: TrainingDAG, uid: str) -> bool:
    n = dag.nodes[uid]
    return n.node_kind == COMPUTE and n.compute_subkind in ("FWD", "BWD", "BWD_I", "BWD_W")


def _ag_preds(dag: TrainingDAG, uid: str) -> list[str]:
    return sorted(e.src_uid for e in dag.in_edges(uid, "data") if dag.nodes[e.src_uid].node_kind == ALL_GATHER)


def _rs_succs(dag: TrainingDAG, uid: str) -> list[str]:
    return sorted(e.dst_uid for e in dag.out_edges(uid, "data") if dag.nodes[e.dst_uid].node_kind == REDUCE_SCATTER)


def _chains(dag: TrainingDAG, candidates: list[str], order: list[str]) -> list[list[str]]:
    pos = {u: i for i, u in enumerate(order)}
    by_bucket: dict[Any, list[str]] = {}
    for u in candidates:
        by_bucket.setdefault(dag.nodes[u].node_meta.get("bucket_key"), []).append(u)
    out: list[list[str]] = []
    for _bucket, uids in sorted(by_bucket.items(), key=lambda kv: str(kv[0])):
        members = set(uids)
        parent = {u: u for u in uids}

        def find(x):
            while parent[x] != x:
                parent[x] = parent[parent[x]]
                x = parent[x]
            return x

        for u in uids:
            for e in dag.out_edges(u):
                if e.tensor_name == STASH_EDGE:
                    continue    # forward -> own backward: not adjacency in time, parameters are released in between
                if e.dst_uid in members:
                    ra, rb = find(u), find(e.dst_uid)
                    if ra != rb:
                        parent[rb] = ra
        groups: dict[str, list[str]] = {}
        for u in uids:
            groups.setdefault(find(u), []).append(u)
        for g in sorted(groups.values(), key=lambda g: min(pos[u] for u in g)):
            out.append(sorted(g, key=pos.get))
    return out


def prune_zero_lifetimes(dag: TrainingDAG) -> list[list[str]]:
    """Prune redundant gathers / reduce-scatters; returns the chains (gradient chains, then parameter chains)."""
    order = serial_topological_order(dag)
    grad_chains: list[list[str]] = []
    param_chains: list[list[str]] = []

    if any(n.node_kind in (REDUCE, REDUCE_SCATTER) for n in dag.nodes.values()):
        cands = [u for u in order if _is_compute(dag, u) and dag.nodes[u].node_meta.get("zero_alloc_full_grads_before")]
        grad_chains = _chains(dag, cands, order)
        for chain in grad_chains:
            for u in chain:
                if not _rs_succs(dag, u):
                    raise AssertionError(f"gradient chain node {u} allocates full grads but has no reduce-scatter")
            for u in chain[1:]:
                dag.nodes[u].node_meta.pop("zero_alloc_full_grads_before", None)
            for u in chain[:-1]:
                for rs in _rs_succs(dag, u):
                    dag.remove_node(rs)
            live = [(u, rs) for u in chain for rs in _rs_succs(dag, u)]
            if not live or any(u != chain[-1] for u, _ in live):
                raise AssertionError(f"only the chain tail may keep a reduce-scatter, got {live}; chain={chain}")

    if any(n.node_kind == ALL_GATHER for n in dag.nodes.values()):
        order = serial_topological_order(dag)
        gathers = {u: _ag_preds(dag, u) for u in order if _is_compute(dag, u)}
        gathers = {u: a for u, a in gathers.items() if a}
        param_chains = _chains(dag, [u for u in order if u in gathers], order)
        for chain in param_chains:
            for u in chain[1:]:
                for ag in gathers[u]:
                    dag.bypass_node(ag)
            for u in chain:
                dag.nodes[u].node_meta.pop("zero_free_full_params_after", None)
                for rs in _rs_succs(dag, u):
                    dag.nodes[rs].node_meta.pop("zero_free_full_params_after", None)
            dag.nodes[chain[-1]].node_meta["zero_free_full_params_after"] = True
            if not _ag_preds(dag, chain[0]):
                raise AssertionError(f"parameter chain root {chain[0]} lost its all-gather")
            for u in chain[1:]:
                if _ag_preds(dag, u):
                    raise AssertionError(f"non-root parameter chain node {u} still has an all-gather")
    return grad_chains + param_chains


def add_inter_chain_temporal_edges(dag: TrainingDAG, chains: list[list[str]]) -> None:
    if not chains:
        return
    levels = dag.topological_levels()

    def maybe(src: str, dst: str) -> None:
        if levels.get(src, 0) < levels.get(dst, 0):
            return
        if dag.has_path(src, dst) or dag.has_path(dst, src):
            return
        dag.connect(src, dst, "temporal")

    params: dict[Any, list[list[str]]] = {}
    grads: dict[Any, list[list[str]]] = {}
    for c in chains:
        b = dag.nodes[c[0]].node_meta.get("bucket_key")
        if _ag_preds(dag, c[0]):
            params.setdefault(b, []).append(c)
        if dag.nodes[c[0]].node_meta.get("zero_alloc_full_grads_before"):
            grads.setdefault(b, []).append(c)
    for cs in params.values():
        cs.sort(key=lambda c: levels.get(c[0], 0))
        for prev, nxt in zip(cs, cs[1:]):
            for ag in _ag_preds(dag, nxt[0]):
                maybe(prev[-1], ag)
    for cs in grads.values():
        cs.sort(key=lambda c: levels.get(c[0], 0))
        for prev, nxt in zip(cs, cs[1:]):
            for rs in _rs_succs(dag, prev[-1]):
                maybe(rs, nxt[0])


_prune_zero_lifetime_metadata = prune_zero_lifetimes
_add_inter_chain_temporal_edges = add_inter_chain_temporal_edges
