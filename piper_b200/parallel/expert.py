"""Expert-parallel token exchange (the A2A tasks that a ``shard`` directive inserts).

True expert parallelism: the experts of a sharded region are partitioned over the group (rank ``r`` owns
experts ``[r*E/ep, (r+1)*E/ep)``) and rows travel to the owner of their expert with per-expert row counts.
The reference exchanges the residual stream with equal splits and keeps every expert on every rank
(``src/executors.py:102-106``, ``src/actor.py:424-448``).

The row buffer entering an exchange is in the padded expert-sorted layout of ``ops.moe``; because experts are
partitioned contiguously, the rows for destination ``d`` are one contiguous block.  The exchange moves the
padded blocks, so the receiver's buffer is again a valid padded layout, now with ``ep * E/ep`` groups ordered
(source rank, local expert), and the received count vector (``[ep * E/ep]``) describes it.  The four exchanges
of one MoE layer and microbatch (dispatch, combine and their gradient mirrors) share the split sizes computed
by the dispatch.

This module is the NCCL/gloo lowering (two small host synchronisations per dispatch to learn the split
sizes); ``parallel/fused.py`` replaces it with kernels that write rows into the owner's memory directly.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

PAD = 128


def _ep_group(executor, node):
    groups = executor.a.groups
    ep = node.node_meta.get("ep_shard") or {}
    ranks = None
    if ep.get("groups"):
        for g in ep["groups"]:
            if executor.a.layout.global_rank in g:
                ranks = list(g)
    if ranks is None:
        ranks = list(ep.get("devices") or executor.a.layout.dp_ranks)
    return (groups.ep_group if groups is not None else None), ranks


def _a2a(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits, group) -> None:
    if group is None:
        out.copy_(inp)
        return
    dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)


def exchange_tokens(executor, node, vals: list) -> tuple:
    """Run the exchange of A2A node ``node`` on the tuple ``vals`` flowing along its edge."""
    m = node.node_meta
    ti = m["a2a_tensor_idx"]
    ci = m.get("a2a_counts_idx")
    group, ranks = _ep_group(executor, node)
    ep = len(ranks)
    is_fwd = node.tag.get("PASS") == "F"
    # an exchange that feeds the expert region (its forward or its backward) moves rows towards the expert owners
    dispatch_dir = m["direction"] == "incoming"
    key = (node.tag.get("MB"), node.tag.get("PP"), node.tag.get("EP"))
    store = executor.a._ep_splits
    rows = vals[ti]
    if rows is None:
        return tuple(vals)
    out_vals = list(vals)

    if is_fwd and m["direction"] == "incoming":
        counts = vals[ci]
        E = counts.numel()
        El = E // ep
        padded = (counts + (PAD - 1)) // PAD * PAD
        if group is not None:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts.contiguous(), group=group)
        else:
            recv_counts = counts.clone()
        recv_padded = (recv_counts + (PAD - 1)) // PAD * PAD
        both = torch.stack((padded.view(ep, El).sum(1), recv_padded.view(ep, El).sum(1))).tolist()
        send_rows, recv_rows = [int(v) for v in both[0]], [int(v) for v in both[1]]
        store[key] = {"send": send_rows, "recv": recv_rows, "cap": rows.shape[0]}
        out = torch.empty((sum(recv_rows), rows.shape[1]), dtype=rows.dtype, device=rows.device)
        _a2a(out, rows[:sum(send_rows)].contiguous(), recv_rows, send_rows, group)
        out_vals[ti] = out
        out_vals[ci] = recv_counts
        return tuple(out_vals)

    info = store[key]
    send_rows, recv_rows, cap = info["send"], info["recv"], info["cap"]
    if dispatch_dir:
        # gradient of the combined rows travelling to the expert owners (backward of the combine exchange)
        out = torch.empty((sum(recv_rows), rows.shape[1]), dtype=rows.dtype, device=rows.device)
        _a2a(out, rows[:sum(send_rows)].contiguous(), recv_rows, send_rows, group)
    else:
        # expert outputs (forward) or row gradients (backward) returning to the token owners
        out = torch.zeros((cap, rows.shape[1]), dtype=rows.dtype, device=rows.device)
        _a2a(out[:sum(send_rows)], rows[:sum(recv_rows)].contiguous(), send_rows, recv_rows, group)
    out_vals[ti] = out
    return tuple(out_vals)
