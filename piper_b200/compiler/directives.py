"""Schedule-directive engine: rewrites a ``TrainingDAG`` according to a directive program.

Directive language (kept byte-compatible with the reference's JSON programs,
``README.md:104-149`` / ``src/directives.py``):

``place``      ``{filter, devices, stream?}``                       assign device sets (compute + UPD)
``replicate``  ``{filter, devices, reduce_stream?, gather_stream?, bucket_size?, shard_grads?, shard_params?}``
``shard``      ``{filter, devices, stream?}``                       expert-parallel region: all-to-all in/out
``split``      ``{filter, dim_name, num_microbatches}``             duplicate a sub-DAG per microbatch
``order``      ``{filters: [[filter, ...], ...]}``                  temporal order of sub-DAGs on one device set

Filters are ``{tag: index | "*"}`` objects, all pairs conjunctive; ``"*"``
matches any non-None index; ``PASS`` is one of F, B, BI, BW.

Application order is fixed and independent of the order in the file:
BI/BW stencil validation -> every ``split`` -> lowering of fused B nodes to
BI + BW where the stencil asks for it -> every ``place`` -> one UPD node per
device set -> SEND/RECV on every cross-device compute edge -> ``replicate`` /
``shard`` in file order -> every ``order``.

Differences from the reference, by design: filter matching runs over a tag
index instead of scanning all nodes for each filter; contiguity checks use
two set traversals per filter instead of two per node (O(N) instead of
O(N^2), ``src/directives.py:1315-1349``); ``shard`` accepts a nested device
list (``[[0,2],[4,6]]``) to make the expert-parallel group a sub-partition of
the data-parallel group.
"""
from __future__ import annotations

from typing import Any, Callable, Iterable, Optional

from .dag import (A2A, ALL_GATHER, COMPUTE, DEFAULT_STREAM, ORDER_DUMMY, RECV, REDUCE, REDUCE_SCATTER, SEND, UPD,
                  TrainingDAG, TrainingDAGEdge, TrainingDAGNode, is_compute, with_pass_tag)

ANY = "__ANY_TAG_INDEX__"
PASSES = ("F", "B", "BI", "BW")
_UID_META_FIELDS = ("fwd_uid", "compute_uid", "bwd_uid", "source_uid", "target_uid", "src_uid", "dst_uid",
                    "from_uid", "to_uid")


# ------------------------------------------------------------------ filters
def normalize_filter(spec: Any, directive: Any = None) -> dict[str, Any]:
    if not isinstance(spec, dict):
        raise ValueError(f"filter must be a JSON object: {directive}")
    out: dict[str, Any] = {}
    for k, v in spec.items():
        if not isinstance(k, str):
            raise ValueError(f"Filter keys must be strings: {directive}")
        if k == "PASS":
            if not isinstance(v, str) or v not in PASSES:
                raise ValueError(f"Invalid 'PASS' filter value {v!r}. Allowed: 'F', 'B', 'BI', 'BW': {directive}")
            out[k] = v
        elif v == "*":
            out[k] = ANY
        elif isinstance(v, str):
            try:
                out[k] = int(v)
            except ValueError:
                out[k] = v
        else:
            out[k] = v
    return out


def match_filter(tag: dict, flt: dict) -> bool:
    for k, v in flt.items():
        if k not in tag:
            return False
        if v == ANY:
            if tag[k] is None:
                return False
        elif tag[k] != v:
            return False
    return True


def _select(dag: TrainingDAG, flt: dict, pred: Optional[Callable[[TrainingDAGNode], bool]] = None) -> list[str]:
    return [u for u, n in dag.nodes.items() if match_filter(n.tag, flt) and (pred is None or pred(n))]


def _schedule_filter_tag_names(directives: Any) -> set[str]:
    if not isinstance(directives, list):
        return set()
    runtime = {"PASS"}
    for d in directives:
        if isinstance(d, dict) and d.get("op") == "split" and isinstance(d.get("dim_name"), str):
            runtime.add(d["dim_name"])
    names: set[str] = set()

    def walk(x):
        if isinstance(x, dict):
            names.update(k for k in x if k not in runtime)
        elif isinstance(x, list):
            for y in x:
                walk(y)

    for d in directives:
        if isinstance(d, dict):
            walk(d.get("filter"))
            walk(d.get("filters"))
    return names


def validate_schedule_tags_exist(dag: TrainingDAG, directives: Any) -> None:
    wanted = _schedule_filter_tag_names(directives)
    if not wanted:
        return
    have = {k for n in dag.nodes.values() for k in n.tag if k != "PASS"}
    missing = sorted(wanted - have)
    if missing:
        raise ValueError("Schedule references tag name(s) not found in model annotations: "
                         f"{missing}. Model tag names: {sorted(have)}.")


# ------------------------------------------------------------------- parsing
def parse_order_directive(directive: Any) -> list[list[dict]]:
    if not isinstance(directive, dict) or directive.get("op") != "order":
        raise ValueError(f"Unsupported order directive: {directive}")
    raw = directive.get("filters")
    if not isinstance(raw, list) or len(raw) < 2:
        raise ValueError(f"order directive requires filters list with at least 2 groups: {directive}")
    groups = []
    for gi, g in enumerate(raw):
        if not isinstance(g, list) or not g:
            raise ValueError(f"order directive filter group[{gi}] must be a non-empty list of filters: {directive}")
        grp = []
        for f in g:
            if not isinstance(f, dict):
                raise ValueError(f"order directive filter group[{gi}] contains invalid filter object: {f}")
            grp.append(normalize_filter(f, directive))
        groups.append(grp)
    return groups


def _parse_device_directive(d: Any) -> dict:
    if not isinstance(d, dict):
        raise ValueError(f"Schedule directives must be JSON objects, got: {type(d)}")
    op = d.get("op")
    if op not in ("place", "replicate", "shard"):
        raise ValueError(f"Unsupported directive op: {op}")
    if "filter" not in d:
        raise ValueError(f"{op} directive requires current API field 'filter': {d}")
    if "filters" in d:
        raise ValueError(f"{op} directive does not accept 'filters': {d}")
    stream, gs, rs = d.get("stream"), d.get("gather_stream"), d.get("reduce_stream")
    if op == "replicate" and stream is not None:
        raise ValueError(f"replicate directive does not accept 'stream'; use 'gather_stream' and/or 'reduce_stream': {d}")
    if op != "replicate" and (gs is not None or rs is not None):
        raise ValueError(f"{op} directive does not accept 'gather_stream'/'reduce_stream'; use 'stream': {d}")
    devices = d.get("devices", d.get("device"))
    if not isinstance(devices, list) or not devices:
        raise ValueError(f"{op} directive requires non-empty devices list: {d}")
    groups = None
    if op == "shard" and all(isinstance(x, list) for x in devices):
        groups = [[int(y) for y in x] for x in devices]
        devices = [y for x in groups for y in x]
    bs = d.get("bucket_size")
    return {
        "op": op, "filter": normalize_filter(d["filter"], d), "devices": [int(x) for x in devices],
        "groups": groups, "stream": None if stream is None else str(stream),
        "gather_stream": None if gs is None else str(gs), "reduce_stream": None if rs is None else str(rs),
        "shard_params": bool(d.get("shard_params", False)), "shard_grads": bool(d.get("shard_grads", False)),
        "bucket_size": None if bs is None else int(bs),
    }


# ------------------------------------------------------- split-backward stencil
def _key_without_pass(flt: dict) -> tuple:
    return tuple(sorted((k, v) for k, v in flt.items() if k != "PASS"))


def validate_split_backward_order_stencil(directives: list) -> set[tuple]:
    """Checks BI/BW entries of all ``order`` rows; returns the tag keys whose B must be split."""
    entries: dict[tuple, list[tuple[int, tuple[int, int], str]]] = {}
    for di, raw in enumerate(directives):
        if not isinstance(raw, dict) or raw.get("op") != "order":
            continue
        seen: dict[tuple, dict[str, tuple]] = {}
        for gi, group in enumerate(parse_order_directive(raw)):
            for fi, flt in enumerate(group):
                p = flt.get("PASS")
                if p not in ("BI", "BW"):
                    continue
                key = _key_without_pass(flt)
                row = seen.setdefault(key, {})
                if p in row:
                    raise ValueError(f"order directive[{di}] has duplicate split-backward {p} entry for "
                                     f"{dict(key)} at indices {row[p]} and {(gi, fi)}")
                row[p] = (gi, fi)
                entries.setdefault(key, []).append((di, (gi, fi), p))
    for key, es in sorted(entries.items(), key=lambda kv: str(kv[0])):
        bi = [e for e in es if e[2] == "BI"]
        bw = [e for e in es if e[2] == "BW"]
        if len(bi) != 1 or len(bw) != 1:
            raise ValueError(f"split backward order entries for {dict(key)} must contain exactly one BI and "
                             f"one BW; got BI={len(bi)} BW={len(bw)}")
        if bi[0][0] != bw[0][0]:
            raise ValueError(f"split backward order entries for {dict(key)} must appear in the same order "
                             "directive row")
        if bi[0][1] > bw[0][1]:
            raise ValueError(f"split backward order entries for {dict(key)} must place BI before BW")
    return set(entries)


def split_fused_bwd_node(dag: TrainingDAG, bwd_uid: str) -> str:
    """B -> BI (same uid) + BW (``{uid}.bw``); UPD now waits on BW."""
    n = dag.nodes[bwd_uid]
    if not is_compute(n, "BWD"):
        raise ValueError(f"expected fused BWD compute node, got {bwd_uid}: {n}")
    w_uid = f"{bwd_uid}.bw"
    if w_uid in dag.nodes:
        raise ValueError(f"duplicate BWD_W uid while splitting {bwd_uid}: {w_uid}")
    n.compute_subkind = "BWD_I"
    n.tag = with_pass_tag(n.tag, "BI")
    meta = dict(n.node_meta)
    meta["compute_loss"] = False
    dag.add_node(TrainingDAGNode(uid=w_uid, node_kind=COMPUTE, compute_subkind="BWD_W",
                                 tag=with_pass_tag(n.tag, "BW"),
                                 device=None if n.device is None else list(n.device), stream=n.stream,
                                 node_meta=meta))
    for e in dag.out_edges(bwd_uid, "temporal"):
        if dag.nodes[e.dst_uid].node_kind == UPD:
            dag.remove_edge(e)
            dag.connect(w_uid, e.dst_uid, "temporal", e.tensor_name)
    dag.connect(bwd_uid, w_uid, "data")
    return w_uid


def apply_split_backward_stencil(dag: TrainingDAG, keys: set[tuple]) -> None:
    if not keys:
        return
    filters = [dict(k) for k in keys]
    for n in list(dag.nodes.values()):
        if is_compute(n, "BWD") and any(match_filter(n.tag, f) for f in filters):
            split_fused_bwd_node(dag, n.uid)


# --------------------------------------------------------------------- split
def apply_split_directive(dag: TrainingDAG, flt: dict, dim_name: str, num_microbatches: int) -> None:
    matched = {u for u in _select(dag, flt) if dag.nodes[u].node_kind != UPD}
    if not matched:
        raise ValueError(f"split(filter={flt}) matched zero nodes")
    topo = dag.topological_order()
    pos = {u: i for i, u in enumerate(topo)}
    lo, hi = min(pos[u] for u in matched), max(pos[u] for u in matched)
    stray = [u for u in topo[lo:hi + 1] if u not in matched and dag.nodes[u].node_kind != UPD]
    if stray:
        raise ValueError(f"split requires a contiguous sub-DAG; found interleaved non-matching nodes: {stray[:8]}")
    sources = {u for u in matched if not (dag.preds[u] & matched)}
    sinks = {u for u in matched if not (dag.succs[u] & matched)}
    incoming, outgoing, inside = [], [], []
    for u in matched:
        for e in dag.in_edges(u):
            (inside if e.src_uid in matched else incoming).append(e)
        for e in dag.out_edges(u):
            if e.dst_uid not in matched:
                outgoing.append(e)
    for e in incoming:
        if dag.nodes[e.src_uid].node_kind != UPD and e.dst_uid not in sources:
            raise ValueError(f"split boundary violation: incoming outside edge targets non-source node {e.dst_uid}")
    for e in outgoing:
        if dag.nodes[e.dst_uid].node_kind != UPD and e.src_uid not in sinks:
            raise ValueError(f"split boundary violation: outgoing outside edge starts at non-sink node {e.src_uid}")
    for u in matched:
        dag.nodes[u].tag[dim_name] = 0
    ordered = [u for u in topo if u in matched]
    for mb in range(1, num_microbatches):
        name = {u: f"{u}.split{dim_name}{mb}" for u in ordered}
        for u in ordered:
            n = dag.nodes[u]
            meta = dict(n.node_meta)
            for k in _UID_META_FIELDS:
                v = meta.get(k)
                if isinstance(v, str) and v in matched:
                    meta[k] = name[v]
            dag.add_node(n.clone(uid=name[u], tag={**n.tag, dim_name: mb}, node_meta=meta))
        for e in inside:
            dag.connect(name[e.src_uid], name[e.dst_uid], e.dep_kind, e.tensor_name)
        for e in incoming:
            dag.connect(e.src_uid, name[e.dst_uid], e.dep_kind, e.tensor_name)
        for e in outgoing:
            dag.connect(name[e.src_uid], e.dst_uid, e.dep_kind, e.tensor_name)


# --------------------------------------------------------------------- place
def device_to_physical_pp_rank(dag: TrainingDAG) -> dict[tuple, int]:
    keys = sorted({n.device_key for n in dag.nodes.values() if n.device is not None})
    return {k: i for i, k in enumerate(keys)}


def replicate_update_nodes_by_device(dag: TrainingDAG) -> None:
    for upd in [n for n in list(dag.nodes.values()) if n.node_kind == UPD and ".rep" not in n.uid]:
        by_dev: dict[tuple, list[TrainingDAGEdge]] = {}
        for e in dag.in_edges(upd.uid, "temporal"):
            src = dag.nodes[e.src_uid]
            if src.device is not None:
                by_dev.setdefault(src.device_key, []).append(e)
        if len(by_dev) <= 1:
            if by_dev:
                upd.device = list(next(iter(by_dev)))
            continue
        outs = dag.out_edges(upd.uid, "temporal")
        for i, (key, edges) in enumerate(sorted(by_dev.items())):
            if i == 0:
                upd.device = list(key)
                continue
            rep = dag.add_node(upd.clone(uid=f"{upd.uid}.rep{i}", device=list(key)))
            for e in edges:
                dag.remove_edge(e)
                dag.connect(e.src_uid, rep.uid, e.dep_kind, e.tensor_name)
            for e in outs:
                dag.connect(rep.uid, e.dst_uid, e.dep_kind, e.tensor_name)


def insert_send_recv_comm_nodes(dag: TrainingDAG, comm_stream: Optional[str] = None) -> None:
    rank_of = device_to_physical_pp_rank(dag)
    n_send = sum(1 for n in dag.nodes.values() if n.node_kind == SEND)
    n_recv = sum(1 for n in dag.nodes.values() if n.node_kind == RECV)
    stream = comm_stream or "pp_stream"
    for e in [e for e in dag.edges if e.dep_kind == "data"]:
        src, dst = dag.nodes[e.src_uid], dag.nodes[e.dst_uid]
        if src.node_kind != COMPUTE or dst.node_kind != COMPUTE:
            continue
        if src.device is None or dst.device is None:
            raise ValueError(f"cannot insert send/recv for unplaced edge {src.uid} -> {dst.uid}")
        if src.device == dst.device:
            continue
        s_uid, r_uid = f"send.{n_send}", f"recv.{n_recv}"
        n_send += 1
        n_recv += 1
        common = {"from_uid": src.uid, "to_uid": dst.uid}
        dag.add_node(TrainingDAGNode(s_uid, SEND, None, dict(src.tag), list(src.device), stream,
                                     {**common, "peer_pp_rank": rank_of[dst.device_key],
                                      "bucket_key": src.node_meta.get("bucket_key"), "pair_uid": r_uid}))
        dag.add_node(TrainingDAGNode(r_uid, RECV, None, dict(dst.tag), list(dst.device), stream,
                                     {**common, "peer_pp_rank": rank_of[src.device_key],
                                      "bucket_key": dst.node_meta.get("bucket_key"), "pair_uid": s_uid}))
        dag.remove_edge(e)
        dag.connect(src.uid, s_uid, "data", e.tensor_name)
        dag.connect(r_uid, dst.uid, "data", e.tensor_name)


# ----------------------------------------------------------------- replicate
def _check_devices(node: TrainingDAGNode, devices: list[int], what: str) -> None:
    if node.device is None:
        raise ValueError(f"{what} requires placed nodes, but node {node.uid} has device=None; "
                         f"expected devices={devices}")
    if sorted(int(d) for d in node.device) != sorted(devices):
        raise ValueError(f"replicate device mismatch for node {node.uid}: expected devices={devices}, "
                         f"node_devices={node.device}")


def _sync_to_update_edges(dag: TrainingDAG, bwd_uid: str, sync_uid: str) -> None:
    """UPD must wait for the gradient sync as well as for the backward itself."""
    for e in dag.out_edges(bwd_uid, "temporal"):
        if dag.nodes[e.dst_uid].node_kind == UPD:
            dag.connect(sync_uid, e.dst_uid, "temporal")


def node_has_trainable_params(dag: TrainingDAG, node: TrainingDAGNode) -> bool:
    meta = node.node_meta
    if is_compute(node, "BWD", "BWD_I", "BWD_W"):
        f = meta.get("fwd_uid")
        if isinstance(f, str) and f in dag.nodes:
            meta = dag.nodes[f].node_meta
    gargs, pidx = meta.get("graphargs"), meta.get("param_idxs")
    if gargs is None or pidx is None:
        return True
    return any(0 <= int(i) < len(gargs) and gargs[int(i)] is not None
               and bool(getattr(gargs[int(i)], "requires_grad", False)) for i in pidx)


def _count(dag: TrainingDAG, kind: str) -> int:
    return sum(1 for n in dag.nodes.values() if n.node_kind == kind)


def insert_reduce_comm_nodes(dag, filters, devices, comm_stream=None) -> None:
    k = _count(dag, REDUCE)
    for n in list(dag.nodes.values()):
        if not is_compute(n, "BWD", "BWD_W") or not any(match_filter(n.tag, f) for f in filters):
            continue
        _check_devices(n, devices, "replicate")
        uid = f"reduce.{k}"
        k += 1
        dag.add_node(TrainingDAGNode(uid, REDUCE, None, dict(n.tag), list(n.device), comm_stream or DEFAULT_STREAM,
                                     {"bwd_uid": n.uid, "bucket_key": n.node_meta.get("bucket_key")}))
        dag.connect(n.uid, uid, "data")
        _sync_to_update_edges(dag, n.uid, uid)


def insert_all_gather_comm_nodes(dag, filters, devices, comm_stream=None) -> None:
    k = _count(dag, ALL_GATHER)
    for n in list(dag.nodes.values()):
        if not is_compute(n, "FWD", "BWD", "BWD_I", "BWD_W") or not any(match_filter(n.tag, f) for f in filters):
            continue
        if not node_has_trainable_params(dag, n):
            continue
        _check_devices(n, devices, "replicate(shard_params=True)")
        uid = f"all_gather.{k}"
        k += 1
        dag.add_node(TrainingDAGNode(uid, ALL_GATHER, None, dict(n.tag), list(n.device),
                                     comm_stream or DEFAULT_STREAM,
                                     {"compute_uid": n.uid, "bucket_key": n.node_meta.get("bucket_key")}))
        n.node_meta["zero_free_full_params_after"] = True
        if n.compute_subkind == "BWD_W":
            for p in sorted(dag.preds[n.uid]):
                if is_compute(dag.nodes[p], "BWD_I"):
                    dag.connect(p, uid, "data")
        dag.connect(uid, n.uid, "data")


def insert_reduce_scatter_comm_nodes(dag, filters, devices, comm_stream=None) -> None:
    k = _count(dag, REDUCE_SCATTER)
    for n in list(dag.nodes.values()):
        if not is_compute(n, "BWD", "BWD_W") or not any(match_filter(n.tag, f) for f in filters):
            continue
        if not node_has_trainable_params(dag, n):
            continue
        _check_devices(n, devices, "replicate(shard_grads/shard_params)")
        uid = f"reduce_scatter.{k}"
        k += 1
        meta = {"bwd_uid": n.uid, "bucket_key": n.node_meta.get("bucket_key")}
        n.node_meta["zero_alloc_full_grads_before"] = True
        if n.node_meta.pop("zero_free_full_params_after", None) is not None:
            meta["zero_free_full_params_after"] = True
        dag.add_node(TrainingDAGNode(uid, REDUCE_SCATTER, None, dict(n.tag), list(n.device),
                                     comm_stream or DEFAULT_STREAM, meta))
        dag.connect(n.uid, uid, "data")
        _sync_to_update_edges(dag, n.uid, uid)


# --------------------------------------------------------------------- shard
def insert_shard_a2a_comm_nodes(dag, filters, devices, comm_stream=None, groups=None) -> None:
    want = sorted(int(d) for d in devices)
    k = _count(dag, A2A)
    sync_kinds = {ALL_GATHER, REDUCE, REDUCE_SCATTER}
    bwd_act = ("BWD", "BWD_I")

    def boundary(src: TrainingDAGNode, dst: TrainingDAGNode) -> dict:
        # a backward edge A.bwd -> B.bwd mirrors the forward edge B -> A, whose
        # producer is the forward node paired with the backward destination
        if is_compute(src, *bwd_act) and is_compute(dst, *bwd_act):
            f = dst.node_meta.get("fwd_uid")
            if not isinstance(f, str) or f not in dag.nodes:
                raise ValueError(f"A2A_COMM could not resolve forward producer for BWD edge "
                                 f"{src.uid}->{dst.uid}: fwd_uid={f!r}")
            producer = dag.nodes[f]
        else:
            producer = src
        info = producer.node_meta.get("a2a_boundary_after")
        if not isinstance(info, dict) or info.get("tensor_idx") is None:
            raise ValueError(f"A2A_COMM missing tensor_idx for edge {src.uid}->{dst.uid}; "
                             f"producer={producer.uid} boundary_info={info!r}")
        return info

    for uid in [u for u, n in dag.nodes.items()
                if n.node_kind == COMPUTE and any(match_filter(n.tag, f) for f in filters)]:
        if uid not in dag.nodes:
            continue
        n = dag.nodes[uid]
        if n.device is None or sorted(int(d) for d in n.device) != want:
            raise ValueError(f"shard requires matched node {uid} to have devices={devices}, got node_devices={n.device}")
        owner = n if n.compute_subkind == "FWD" else dag.nodes.get(n.node_meta.get("fwd_uid"), None)
        if owner is not None:
            owner.node_meta["apply_zero"] = False
            owner.node_meta["ep_shard"] = {"devices": list(devices), "groups": groups}
        n.node_meta["ep_shard"] = {"devices": list(devices), "groups": groups}
        # expert parameters are partitioned, not replicated: drop the DP sync
        # comms that an earlier replicate attached to this node
        attached = sorted({e.dst_uid for e in dag.out_edges(uid, "data") if dag.nodes[e.dst_uid].node_kind in sync_kinds}
                          | {e.src_uid for e in dag.in_edges(uid, "data") if dag.nodes[e.src_uid].node_kind in sync_kinds})
        for c in attached:
            dag.bypass_node(c)
        if attached:
            n.node_meta.pop("zero_alloc_full_grads_before", None)
            n.node_meta.pop("zero_free_full_params_after", None)
        if n.compute_subkind == "BWD_W":
            continue

        def same_pass_compute(e: TrainingDAGEdge) -> bool:
            a, b = dag.nodes[e.src_uid], dag.nodes[e.dst_uid]
            if a.node_kind != COMPUTE or b.node_kind != COMPUTE:
                return False
            if n.compute_subkind == "FWD":
                return a.compute_subkind == "FWD" and b.compute_subkind == "FWD"
            return is_compute(a, *bwd_act) and is_compute(b, *bwd_act)

        incoming = [e for e in dag.in_edges(uid, "data") if same_pass_compute(e)]
        outgoing = [e for e in dag.out_edges(uid, "data") if same_pass_compute(e)]
        for e, other_uid, side in ([(e, e.src_uid, "incoming") for e in incoming]
                                   + [(e, e.dst_uid, "outgoing") for e in outgoing]):
            o = dag.nodes[other_uid]
            if o.device is None or sorted(int(d) for d in o.device) != want:
                raise ValueError(f"shard precondition failed for {side} edge {e.src_uid}->{e.dst_uid}: "
                                 f"neighbour compute must be replicated on devices={devices}, got {o.device}")
            if o.tag.get("PASS") != n.tag.get("PASS"):
                raise ValueError(f"A2A_COMM requires matching compute pass tags; {side} edge "
                                 f"{e.src_uid}->{e.dst_uid} has PASS {o.tag.get('PASS')} vs {n.tag.get('PASS')}")
        for e in incoming:
            info = boundary(dag.nodes[e.src_uid], n)
            c = f"a2a.{k}"
            k += 1
            dag.add_node(TrainingDAGNode(c, A2A, None, dict(n.tag), list(n.device), comm_stream or DEFAULT_STREAM,
                                         {"direction": "incoming", "target_uid": uid,
                                          "a2a_tensor_idx": info["tensor_idx"],
                                          "a2a_counts_idx": info.get("counts_idx"),
                                          "ep_shard": {"devices": list(devices), "groups": groups},
                                          "bucket_key": n.node_meta.get("bucket_key")}))
            dag.remove_edge(e)
            dag.connect(e.src_uid, c, "data", e.tensor_name)
            dag.connect(c, uid, "data", e.tensor_name)
        for e in outgoing:
            info = boundary(n, dag.nodes[e.dst_uid])
            c = f"a2a.{k}"
            k += 1
            dag.add_node(TrainingDAGNode(c, A2A, None, dict(n.tag), list(n.device), comm_stream or DEFAULT_STREAM,
                                         {"direction": "outgoing", "source_uid": uid,
                                          "a2a_tensor_idx": info["tensor_idx"],
                                          "a2a_counts_idx": info.get("counts_idx"),
                                          "ep_shard": {"devices": list(devices), "groups": groups},
                                          "bucket_key": n.node_meta.get("bucket_key")}))
            dag.remove_edge(e)
            dag.connect(uid, c, "data", e.tensor_name)
            dag.connect(c, e.dst_uid, "data", e.tensor_name)


# ------------------------------------------------------------------ bucketing
def bucket_matched_fwd_nodes(dag: TrainingDAG, filters: list[dict], bucket_size_mb: int,
                             bucket_stage_fn: Optional[Callable] = None) -> None:
    """Replace FWD/BWD pairs by chains of per-parameter-bucket nodes (``replicate.bucket_size``)."""
    if bucket_size_mb <= 0:
        raise ValueError(f"bucket_size must be > 0 MB, got {bucket_size_mb}")
    if bucket_stage_fn is None:
        from . import bucket as _bucket
        bucket_stage_fn = _bucket.bucket_stage
    limit = int(bucket_size_mb) * 1024 * 1024
    targets = [u for u, n in dag.nodes.items() if is_compute(n, "FWD") and any(match_filter(n.tag, f) for f in filters)]
    targets.sort(key=lambda u: (int(dag.nodes[u].node_meta.get("stage_id", 10 ** 9)),
                                int(dag.nodes[u].node_meta.get("segment_id", 10 ** 9)),
                                int(dag.nodes[u].tag.get("MB", 0) or 0)))
    plan_cache: dict[int, list] = {}
    for f_uid in targets:
        fn = dag.nodes[f_uid]
        bwds = sorted(u for u, n in dag.nodes.items() if is_compute(n, "BWD") and n.node_meta.get("fwd_uid") == f_uid)
        if len(bwds) != 1:
            raise ValueError(f"Expected exactly one fused BWD node for {f_uid}, found {bwds}")
        b_uid = bwds[0]
        bn = dag.nodes[b_uid]
        m = fn.node_meta
        gm = m.get("gm")
        if gm is None or m.get("graphargs") is None or m.get("input_idxs") is None or m.get("param_idxs") is None:
            continue
        key = id(gm)
        if key not in plan_cache:
            plan_cache[key] = bucket_stage_fn(gm, m["graphargs"], m["input_idxs"], m["param_idxs"],
                                              bucket_size_bytes=limit, debug_name=f_uid)
        buckets = plan_cache[key]
        if len(buckets) <= 1:
            continue
        in_f, out_f = dag.in_edges(f_uid), dag.out_edges(f_uid)
        in_b, out_b = dag.in_edges(b_uid), dag.out_edges(b_uid)
        f_chain, b_chain = [], []
        fqns = m.get("param_fqns") or []
        for i, bucket in enumerate(buckets):
            bgm, b_in, b_par, b_args = bucket[:4]
            b_fqns = bucket[4] if len(bucket) > 4 else []
            fu = f"{f_uid}.bucket{i}"
            bkey = f"{m.get('bucket_key', f_uid)}.bucket{i}"     # shared by all microbatch copies
            f_chain.append(fu)
            b_chain.append(f"{fu}.bwd")
            dag.add_node(TrainingDAGNode(fu, COMPUTE, "FWD", with_pass_tag(fn.tag, "F"),
                                         None if fn.device is None else list(fn.device), fn.stream, {
                "stage_id": int(m.get("stage_id", -1)), "segment_id": int(m.get("segment_id", -1)) * 1000 + i,
                "gm": bgm, "input_idxs": list(b_in), "param_idxs": list(b_par), "graphargs": list(b_args),
                "param_fqns": list(b_fqns) if b_fqns else [],
                "input_names": [x.name for x in bgm.graph.nodes if x.op == "placeholder"], "output_names": [],
                "a2a_boundary_after": m.get("a2a_boundary_after") if i == len(buckets) - 1 else None,
                "bucket_idx": i, "num_buckets": len(buckets), "bucket_key": bkey, "parent_uid": f_uid}))
            dag.add_node(TrainingDAGNode(f"{fu}.bwd", COMPUTE, "BWD", with_pass_tag(fn.tag, "B"),
                                         None if bn.device is None else list(bn.device), bn.stream, {
                "fwd_uid": fu, "bucket_idx": i, "num_buckets": len(buckets), "bucket_key": bkey,
                "compute_loss": bool(bn.node_meta.get("compute_loss", False)) and i == len(buckets) - 1}))
        del fqns
        first_f, last_f, first_b, last_b = f_chain[0], f_chain[-1], b_chain[-1], b_chain[0]
        remap = {f_uid: last_f, b_uid: first_b}
        dag.remove_node(f_uid)
        dag.remove_node(b_uid)
        for e in in_f:
            dag.connect(remap.get(e.src_uid, e.src_uid), first_f, e.dep_kind, e.tensor_name)
        for e in out_f:
            dag.connect(last_f, first_b if e.dst_uid == b_uid else e.dst_uid, e.dep_kind, e.tensor_name)
        for e in in_b:
            dag.connect(remap.get(e.src_uid, e.src_uid), first_b, e.dep_kind, e.tensor_name)
        for e in out_b:
            dag.connect(last_b, remap.get(e.dst_uid, e.dst_uid), e.dep_kind, e.tensor_name)
        for a, b in zip(f_chain, f_chain[1:]):
            dag.connect(a, b, "data")
        for a, b in zip(reversed(b_chain), list(reversed(b_chain))[1:]):
            dag.connect(a, b, "data")
        # pipeline messages were attached to the nodes this chain replaces: a send now leaves from the end of the
        # forward (backward) chain and a receive feeds its head
        for other in dag.nodes.values():
            if other.node_kind in (SEND, RECV):
                om = other.node_meta
                if om.get("from_uid") in (f_uid, b_uid):
                    om["from_uid"] = last_f if om["from_uid"] == f_uid else last_b
                if om.get("to_uid") in (f_uid, b_uid):
                    om["to_uid"] = first_f if om["to_uid"] == f_uid else first_b
        # every bucket's backward gates the update
        for e in out_b:
            if e.dep_kind == "temporal" and dag.nodes[e.dst_uid].node_kind == UPD:
                for b in b_chain:
                    dag.connect(b, e.dst_uid, "temporal")


# --------------------------------------------------------------------- order
def match_set_contiguous_subdag(dag: TrainingDAG, matched: set[str], *, context: str):
    """Returns (sources, sinks, compute_sources, compute_sinks) of a matched set that must be contiguous."""
    if not matched:
        raise ValueError(f"{context}: filter matched zero nodes")
    # a non-matching node lies "between" matched nodes iff it has both a
    # matched ancestor and a matched descendant
    below: set[str] = set()
    stack = list(matched)
    while stack:
        for v in dag.succs[stack.pop()]:
            if v not in below:
                below.add(v)
                stack.append(v)
    above: set[str] = set()
    stack = list(matched)
    while stack:
        for v in dag.preds[stack.pop()]:
            if v not in above:
                above.add(v)
                stack.append(v)
    between = [u for u in dag.nodes if u not in matched and u in below and u in above]
    if between:
        raise ValueError(f"{context}: matched nodes are not contiguous; interleaved non-matching nodes: {between[:8]}")
    sources = {u for u in matched if not (dag.preds[u] & matched)}
    sinks = {u for u in matched if not (dag.succs[u] & matched)}
    if not sources or not sinks:
        raise ValueError(f"{context}: failed to identify non-empty source/sink sets")
    compute = {u for u in matched if dag.nodes[u].node_kind == COMPUTE}

    def reaches_compute(u: str, nbrs) -> bool:
        seen = {u}
        st = [v for v in nbrs[u] if v in matched]
        while st:
            c = st.pop()
            if c in seen:
                continue
            seen.add(c)
            if c in compute:
                return True
            st.extend(v for v in nbrs[c] if v in matched)
        return False

    csrc = {u for u in compute if not reaches_compute(u, dag.preds)}
    csnk = {u for u in compute if not reaches_compute(u, dag.succs)}
    if not csrc or not csnk:
        raise ValueError(f"{context}: failed to identify non-empty compute source/sink sets")
    return sources, sinks, csrc, csnk


def _order_edge(dag: TrainingDAG, src: str, dst: str, di: int) -> None:
    if dag.has_path(dst, src):
        raise ValueError(f"order directive[{di}] violates model dataflow: adding temporal edge "
                         f"{src} -> {dst} would create a cycle")
    a, b = dag.nodes[src].device_key, dag.nodes[dst].device_key
    if a is None or b is None:
        raise ValueError(f"order directive[{di}] requires placed nodes with a single device set: "
                         f"{src} device={a}, {dst} device={b}")
    if a != b:
        raise ValueError(f"order directive[{di}] crosses device placement: {src} device={a}, {dst} device={b}")
    dag.connect(src, dst, "temporal")


def apply_order_directive(dag: TrainingDAG, filter_groups: list[list[dict]], *, directive_idx: int) -> None:
    segments: list[tuple[set[str], set[str]]] = []
    for gi, group in enumerate(filter_groups):
        srcs, snks, members = [], [], set()
        for fi, flt in enumerate(group):
            matched = set(_select(dag, flt, lambda n: n.node_kind != ORDER_DUMMY))
            _, _, cs, ck = match_set_contiguous_subdag(dag, matched, context=f"order filter[{gi}][{fi}]={flt}")
            srcs.append(cs)
            snks.append(ck)
            members |= matched
        if len(group) == 1:
            segments.append((srcs[0], snks[0]))
            continue
        devs = {tuple(dag.nodes[u].device) for u in members if dag.nodes[u].device is not None}
        dev = list(next(iter(devs))) if len(devs) == 1 else None
        s_uid = f"order.{directive_idx}.group{gi}.source"
        k_uid = f"order.{directive_idx}.group{gi}.sink"
        for uid, role in ((s_uid, "source"), (k_uid, "sink")):
            dag.add_node(TrainingDAGNode(uid, ORDER_DUMMY, None, {"order": directive_idx, "group": gi}, dev,
                                         DEFAULT_STREAM, {"role": role}))
        for cs in srcs:
            for v in sorted(cs):
                _order_edge(dag, s_uid, v, directive_idx)
        for ck in snks:
            for u in sorted(ck):
                _order_edge(dag, u, k_uid, directive_idx)
        segments.append(({s_uid}, {k_uid}))
    for (_, snk), (src, _) in zip(segments, segments[1:]):
        for u in sorted(snk):
            for v in sorted(src):
                _order_edge(dag, u, v, directive_idx)


# -------------------------------------------------------------------- driver
def apply_schedule_directives(dag: TrainingDAG, directives: Optional[list]) -> None:
    if not directives:
        return
    stencil = validate_split_backward_order_stencil(directives)
    for raw in directives:
        if isinstance(raw, dict) and raw.get("op") == "split":
            dim = raw.get("dim_name")
            if not isinstance(dim, str) or not dim:
                raise ValueError(f"split directive requires non-empty string dim_name: {raw}")
            n = int(raw.get("num_microbatches", 0))
            if n <= 0:
                raise ValueError(f"split directive requires num_microbatches > 0: {raw}")
            apply_split_directive(dag, normalize_filter(raw.get("filter"), raw), dim, n)
    apply_split_backward_stencil(dag, stencil)

    place_streams: set[str] = set()
    for i, raw in enumerate(directives):
        if not isinstance(raw, dict) or raw.get("op") != "place":
            continue
        d = _parse_device_directive(raw)
        hit = 0
        for n in dag.nodes.values():
            if n.node_kind in (COMPUTE, UPD) and match_filter(n.tag, d["filter"]):
                n.device = list(d["devices"])
                hit += 1
        if hit == 0:
            raise ValueError(f"place directive[{i}] matched zero nodes: {raw}")
        if d["stream"] is not None:
            place_streams.add(d["stream"])
    if len(place_streams) > 1:
        raise ValueError(f"place directives must agree on stream, got {sorted(place_streams)}")
    replicate_update_nodes_by_device(dag)
    insert_send_recv_comm_nodes(dag, comm_stream=next(iter(place_streams), None))

    for i, raw in enumerate(directives):
        if not isinstance(raw, dict) or raw.get("op") not in ("replicate", "shard"):
            continue
        d = _parse_device_directive(raw)
        flts = [d["filter"]]
        if not _select(dag, d["filter"], lambda n: n.node_kind == COMPUTE):
            raise ValueError(f"{d['op']} directive[{i}] matched zero compute nodes: {raw}")
        if d["op"] == "replicate":
            if d["bucket_size"] is not None:
                bucket_matched_fwd_nodes(dag, flts, d["bucket_size"])
            if d["shard_params"]:
                insert_all_gather_comm_nodes(dag, flts, d["devices"], d["gather_stream"])
                insert_reduce_scatter_comm_nodes(dag, flts, d["devices"], d["reduce_stream"])
            elif d["shard_grads"]:
                insert_reduce_scatter_comm_nodes(dag, flts, d["devices"], d["reduce_stream"])
            else:
                insert_reduce_comm_nodes(dag, flts, d["devices"], d["reduce_stream"])
        else:
            insert_shard_a2a_comm_nodes(dag, flts, d["devices"], d["stream"], d["groups"])

    for i, raw in enumerate(directives):
        if isinstance(raw, dict) and raw.get("op") == "order":
            apply_order_directive(dag, parse_order_directive(raw), directive_idx=i)


# reference-compatible private names (its tests and the `src.piper` shim use them)
_match_filter = match_filter
_normalize_filter_spec = normalize_filter
_parse_order_directive = parse_order_directive
_validate_split_backward_order_stencil = validate_split_backward_order_stencil
_apply_split_backward_stencil = apply_split_backward_stencil
_split_fused_bwd_node = split_fused_bwd_node
_apply_split_directive = apply_split_directive
_apply_order_directive = apply_order_directive
_validate_schedule_tags_exist = validate_schedule_tags_exist
_insert_reduce_scatter_comm_nodes = insert_reduce_scatter_comm_nodes
_insert_shard_a2a_comm_nodes = insert_shard_a2a_comm_nodes
_insert_reduce_comm_nodes = insert_reduce_comm_nodes
_insert_all_gather_comm_nodes = insert_all_gather_comm_nodes
_insert_send_recv_comm_nodes = insert_send_recv_comm_nodes
_replicate_update_nodes_by_device = replicate_update_nodes_by_device
_match_set_contiguous_subdag = match_set_contiguous_subdag


def _bucket_matched_fwd_nodes(dag, filters, bucket_size_mb):
    import sys
    mod = sys.modules[__name__]
    return bucket_matched_fwd_nodes(dag, filters, bucket_size_mb, getattr(mod, "bucket_stage", None))
