"""Parameter bucketing of one stage graph (``replicate.bucket_size``).

``bucket_stage`` cuts a stage's ``GraphModule`` into consecutive sub-graphs so that each reads at most
``bucket_size_bytes`` of trainable parameters; the directive engine then replaces the stage's FWD/BWD pair by
a chain of per-bucket nodes, so that a bucket's gradient synchronisation can start as soon as its own
backward has finished instead of after the whole stage.  Rules (the reference states the same ones,
``src/bucket.py:15-360``, but its implementation raises on every plan with more than one bucket):

* greedy fill in execution order: a cut is placed before the first op whose new parameters would overflow
  the current bucket;
* a parameter belongs to exactly one bucket: buckets spanned by the uses of one parameter are merged;
* no cut may be crossed by a *view* of a parameter (``t``, ``view``, ``reshape``, ``permute``, ...): the
  alias would carry parameter storage into another bucket's lifetime, so the two buckets are merged.

The sub-graphs themselves are produced by the ordinary segment splitter, with the bucket index as the
annotation, so bucket graphs and segment graphs obey one placeholder contract.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.fx as fx

from .fxsplit import PIPER_ANNOTATIONS_META_KEY, example_value, split_gm_by_annotations

_VIEW_NAMES = {"t", "transpose", "view", "reshape", "permute", "expand", "detach", "alias", "squeeze", "unsqueeze",
               "getitem", "contiguous", "flatten", "unflatten", "narrow", "select", "T", "mT", "to", "_to_copy"}


def _op_name(n: fx.Node) -> str:
    t = n.target
    if isinstance(t, str):
        return t
    name = getattr(t, "__name__", None) or str(t)
    return name.split(".")[-1] if "." in name and not hasattr(t, "__name__") else name


def _is_param_alias(n: fx.Node, params: set, memo: dict) -> bool:
    """True when ``n`` is a chain of view-like ops over a single parameter placeholder."""
    if n in memo:
        return memo[n]
    res = False
    if n in params:
        res = True
    elif n.op in ("call_function", "call_method") and _op_name(n).split(".")[0] in _VIEW_NAMES:
        ins = [i for i in n.all_input_nodes]
        res = len(ins) >= 1 and all(_is_param_alias(i, params, memo) for i in ins[:1]) and \
            all(i in params or _is_param_alias(i, params, memo) for i in ins)
    memo[n] = res
    return res


def plan_buckets(gm: fx.GraphModule, graphargs: list, param_idxs: list, bucket_size_bytes: int) -> list[int]:
    """Bucket index of every compute node of ``gm`` (in graph order)."""
    nodes = list(gm.graph.nodes)
    phs = [n for n in nodes if n.op == "placeholder"]
    compute = [n for n in nodes if n.op not in ("placeholder", "get_attr", "output")]
    trainable = {}
    for i in param_idxs:
        g = graphargs[i]
        if i < len(phs) and isinstance(g, torch.Tensor) and bool(getattr(g, "requires_grad", False)):
            trainable[phs[i]] = int(g.numel()) * int(g.element_size())
    params = {phs[i] for i in param_idxs if i < len(phs)}
    pos = {n: i for i, n in enumerate(compute)}
    # 1. greedy fill
    assign, cur, fill, seen = [], 0, 0, set()
    for n in compute:
        new = sum(b for p, b in trainable.items() if p in n.all_input_nodes and p not in seen)
        if fill > 0 and new > 0 and fill + new > bucket_size_bytes:
            cur += 1
            fill = 0
        for p in n.all_input_nodes:
            if p in trainable and p not in seen:
                seen.add(p)
        fill += new
        assign.append(cur)
    # 2./3. merge buckets that share a parameter or are connected by a parameter alias
    parent = list(range(cur + 1))

    def find(x):
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    def merge_range(a, b):
        lo, hi = min(a, b), max(a, b)
        for k in range(lo, hi):
            ra, rb = find(k), find(k + 1)
            if ra != rb:
                parent[max(ra, rb)] = min(ra, rb)

    for p in params:
        used = [assign[pos[u]] for u in p.users if u in pos]
        if used:
            merge_range(min(used), max(used))
    memo: dict = {}
    for n in compute:
        if _is_param_alias(n, params, memo):
            for u in n.users:
                if u in pos and assign[pos[u]] != assign[pos[n]]:
                    merge_range(assign[pos[n]], assign[pos[u]])
    roots = sorted({find(b) for b in range(cur + 1)})
    dense = {r: i for i, r in enumerate(roots)}
    return [dense[find(b)] for b in assign]


def bucket_stage(gm: fx.GraphModule, graphargs: list, input_idxs: list, param_idxs: list, *,
                 bucket_size_bytes: int, debug_name: str = "") -> list[tuple]:
    """Returns ``[(bucket_gm, input_idxs, param_idxs, graphargs, param_fqns), ...]`` in execution order."""
    assign = plan_buckets(gm, graphargs, param_idxs, bucket_size_bytes)
    if not assign or max(assign) == 0:
        return [(gm, list(input_idxs), list(param_idxs), list(graphargs), [])]
    nodes = list(gm.graph.nodes)
    phs = [n for n in nodes if n.op == "placeholder"]
    compute = [n for n in nodes if n.op not in ("placeholder", "get_attr", "output")]
    saved = []
    for n, b in zip(compute, assign):
        custom = n.meta.get("custom")
        saved.append((n, None if custom is None else dict(custom)))
        n.meta["custom"] = {PIPER_ANNOTATIONS_META_KEY: ({"name": "BUCKET", "index": int(b), "uid": int(b)},)}
    try:
        runtime = {phs[i].name for i in input_idxs}
        _, segs = split_gm_by_annotations(gm, runtime_input_names=runtime)
    finally:
        for n, custom in saved:
            if custom is None:
                n.meta.pop("custom", None)
            else:
                n.meta["custom"] = custom
    return [(s.gm, list(s.input_idxs), list(s.param_idxs), list(s.graphargs), list(s.param_fqns)) for s in segs]
