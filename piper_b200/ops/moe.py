"""Mixture-of-experts ops: router, dispatch into padded expert segments, grouped linear, combine.

Row layout.  ``moe_dispatch`` copies each token once per selected expert into a row buffer in which the
entries of expert ``e`` occupy rows ``[g_start[e], g_start[e] + counts[e])``; every segment is padded with
zero rows to a multiple of 128 (``g_len``), so a segment is a whole number of tensor-core M tiles and the
weight-gradient GEMM can contract over padded segments.  The grouped linear op takes such a buffer plus a
*group table* ``(g_start, g_len)`` with ``G = sources * experts`` groups, group ``g`` using expert
``g % experts``; ``sources`` is 1 without expert parallelism and the expert-parallel degree after a token
exchange, when rows arrive grouped by (source rank, local expert).

The reference's expert compute pads every expert to ``T*k`` rows and runs ``bmm``
(``examples/models/qwen3_bmm_experts_patch.py:24-37``, an ``E``-fold waste); its un-permute and weighted
combine are separate index-put / ``bmm`` calls (``examples/models/qwen3.py:265-283``).  Here dispatch,
combine and their gradients are one kernel each and the expert GEMMs are ragged.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import core, native
from .core import _is_native, _require_bf16, grad_sinks, wgrad_store

PAD = 128

# Set by the executor around a segment run when the expert-parallel exchanges are lowered to peer-memory kernels
# (``parallel/ep_fused.py``): ``_EP_RUNTIME.dispatch`` replaces the local permutation of ``moe_dispatch`` by a
# gather straight into the expert owners' receive regions, and ``_EP_TABLE`` is the group table of the receive
# region that the expert segment reads in place.
_EP_RUNTIME = None
_EP_TABLE = None


def set_ep_context(runtime, table) -> None:
    global _EP_RUNTIME, _EP_TABLE
    _EP_RUNTIME, _EP_TABLE = runtime, table


def row_capacity(tokens: int, k: int, experts: int) -> int:
    """Rows a dispatch buffer needs in the worst case (every segment padded by up to PAD-1 rows)."""
    return (tokens * k + experts * (PAD - 1) + PAD - 1) // PAD * PAD


# ------------------------------------------------------------------ router
@torch.library.custom_op("piper::moe_route", mutates_args=())
def moe_route(logits: Tensor, k: int, renorm: bool) -> tuple[Tensor, Tensor, Tensor]:
    """softmax over experts, top-k, optional renormalisation -> (weights fp32 [T,k], idx int32 [T,k], counts int32 [E])."""
    T, E = logits.shape
    if _is_native(logits):
        _require_bf16(logits)
        w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
        idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
        counts = torch.zeros(E, dtype=torch.int32, device=logits.device)
        native.lib().moe_route(logits.contiguous(), w, idx, counts, k, renorm)
        return w, idx, counts
    p = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(p, k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    counts = torch.bincount(idx.reshape(-1), minlength=E).to(torch.int32)
    return w.contiguous(), idx.to(torch.int32).contiguous(), counts


@moe_route.register_fake
def _(logits, k, renorm):
    T, E = logits.shape
    return (logits.new_empty((T, k), dtype=torch.float32), logits.new_empty((T, k), dtype=torch.int32),
            logits.new_empty((E,), dtype=torch.int32))


def _route_setup(ctx, inputs, output):
    logits, k, renorm = inputs
    w, idx, _counts = output
    ctx.renorm = renorm
    ctx.save_for_backward(logits, idx, w)


def _route_backward(ctx, dw, _didx, _dcounts):
    logits, idx, w = ctx.saved_tensors
    if _is_native(logits):
        d = torch.empty_like(logits, memory_format=torch.contiguous_format)
        native.lib().moe_route_bwd(logits.contiguous(), idx, w, dw.contiguous().float(), d, ctx.renorm)
        return d, None, None
    p = torch.softmax(logits.float(), dim=-1)
    dp = torch.zeros_like(p)
    g = dw.float()
    if ctx.renorm:
        S = torch.gather(p, 1, idx.long()).sum(-1, keepdim=True)
        g = (g - (g * w).sum(-1, keepdim=True)) / S
    dp.scatter_(1, idx.long(), g)
    d = p * (dp - (dp * p).sum(-1, keepdim=True))
    return d.to(logits.dtype), None, None


moe_route.register_autograd(_route_backward, setup_context=_route_setup)


# -------------------------------------------------------------- group table
@torch.library.custom_op("piper::moe_group_table", mutates_args=())
def moe_group_table(counts: Tensor, expert_weights: Tensor) -> tuple[Tensor, Tensor]:
    """counts [G] int32 (source-major) -> (g_start, g_len): padded segments laid out back to back.

    The number of local experts is read from ``expert_weights.shape[0]`` when the op runs, not baked in as a
    traced constant, so the same graph serves any expert-parallel degree.
    """
    experts = expert_weights.shape[0]
    if _is_native(counts):
        if _EP_TABLE is not None and _EP_TABLE[0].numel() == counts.numel():
            return _EP_TABLE[0].clone(), _EP_TABLE[1].clone()
        g_start = torch.empty_like(counts)
        g_len = torch.empty_like(counts)
        total = torch.empty(1, dtype=torch.int32, device=counts.device)
        native.lib().moe_group_table(counts.contiguous(), experts, None, g_start, g_len, total)
        return g_start, g_len
    g_len = (counts + (PAD - 1)) // PAD * PAD
    g_start = torch.cumsum(g_len, 0) - g_len
    return g_start.to(torch.int32), g_len.to(torch.int32)


@moe_group_table.register_fake
def _(counts, expert_weights):
    return torch.empty_like(counts), torch.empty_like(counts)


# ---------------------------------------------------------------- dispatch
@torch.library.custom_op("piper::moe_dispatch", mutates_args=())
def moe_dispatch(x: Tensor, idx: Tensor, counts: Tensor) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """x [T, D] -> (rows [cap, D], pos int32 [T*k], g_start int32 [E], g_len int32 [E], ep_counts int32 [E]).

    ``ep_counts`` is a copy of ``counts`` meant for the expert region alone: an expert-parallel token exchange
    replaces it by the counts received from the peers, while ``counts`` keeps describing the local layout.
    """
    T, D = x.shape
    k = idx.shape[1]
    E = counts.shape[0]
    cap = row_capacity(T, k, E)
    if _is_native(x):
        _require_bf16(x)
        if _EP_RUNTIME is not None and _EP_RUNTIME.active is not None:
            return _EP_RUNTIME.dispatch(x, idx, counts)
        g_start = torch.empty_like(counts)
        g_len = torch.empty_like(counts)
        total = torch.empty(1, dtype=torch.int32, device=x.device)
        native.lib().moe_group_table(counts, E, None, g_start, g_len, total)
        rows = torch.empty((cap, D), dtype=x.dtype, device=x.device)
        pos = torch.empty(T * k, dtype=torch.int32, device=x.device)
        cursor = torch.zeros(E, dtype=torch.int32, device=x.device)
        native.lib().moe_permute(x.contiguous(), idx, g_start, g_len, counts, cursor, pos, rows)
        return rows, pos, g_start, g_len, counts.clone()
    g_len = (counts + (PAD - 1)) // PAD * PAD
    g_start = (torch.cumsum(g_len, 0) - g_len).to(torch.int32)
    flat_e = idx.reshape(-1).long()
    order = torch.argsort(flat_e, stable=True)
    rank_in_e = torch.empty_like(order)
    sorted_e = flat_e[order]
    first = torch.searchsorted(sorted_e, sorted_e)
    rank_in_e[order] = torch.arange(order.numel()) - first
    pos = (g_start.long()[flat_e] + rank_in_e).to(torch.int32)
    rows = torch.zeros((cap, D), dtype=x.dtype)
    rows[pos.long()] = x.repeat_interleave(k, dim=0)
    return rows, pos, g_start, g_len.to(torch.int32), counts.clone()


@moe_dispatch.register_fake
def _(x, idx, counts):
    T, D = x.shape
    k, E = idx.shape[1], counts.shape[0]
    return (x.new_empty((row_capacity(T, k, E), D)), x.new_empty((T * k,), dtype=torch.int32),
            torch.empty_like(counts), torch.empty_like(counts), torch.empty_like(counts))


def _dispatch_setup(ctx, inputs, output):
    x, idx, _counts = inputs
    ctx.k = idx.shape[1]
    ctx.xshape = x.shape
    ctx.save_for_backward(output[1])


def _dispatch_backward(ctx, drows, _dpos, _dgs, _dgl, _dec):
    (pos,) = ctx.saved_tensors
    T, D = ctx.xshape
    if _is_native(drows):
        dx = torch.empty((T, D), dtype=drows.dtype, device=drows.device)
        native.lib().moe_permute_bwd(drows.contiguous(), pos, dx, ctx.k)
        return dx, None, None
    dx = drows[pos.long()].float().reshape(T, ctx.k, D).sum(1)
    return dx.to(drows.dtype), None, None


moe_dispatch.register_autograd(_dispatch_backward, setup_context=_dispatch_setup)


# ----------------------------------------------------------- grouped linear
def _grouped(mode: int, x, dy, w, out, g_start, g_len, experts: int, N: int, K: int, accumulate: bool = False):
    native.lib().grouped_gemm(mode, x, dy, w, out, g_start, g_len, experts, N, K, accumulate,
                              native.status_tensor(out.device))
    return out


def _grouped_ref_segments(g_start: Tensor, g_len: Tensor):
    gs, gl = g_start.tolist(), g_len.tolist()
    return [(g, s, s + n) for g, (s, n) in enumerate(zip(gs, gl)) if n > 0]


@torch.library.custom_op("piper::grouped_linear", mutates_args=())
def grouped_linear(rows: Tensor, w: Tensor, g_start: Tensor, g_len: Tensor) -> Tensor:
    """out[r] = rows[r] @ w[expert(group of r)]^T for w [experts, N, K]; rows outside every group are undefined."""
    E, N, K = w.shape
    if _is_native(rows):
        _require_bf16(rows, w)
        out = torch.empty((rows.shape[0], N), dtype=rows.dtype, device=rows.device)
        return _grouped(0, rows.contiguous(), None, w, out, g_start, g_len, E, N, K)
    out = torch.zeros((rows.shape[0], N), dtype=rows.dtype)
    for g, a, b in _grouped_ref_segments(g_start, g_len):
        out[a:b] = rows[a:b] @ w[g % E].t()
    return out


@grouped_linear.register_fake
def _(rows, w, g_start, g_len):
    return rows.new_empty((rows.shape[0], w.shape[1]))


def _grouped_wgrad(rows: Tensor, dy: Tensor, w: Tensor, g_start: Tensor, g_len: Tensor) -> Optional[Tensor]:
    E, N, K = w.shape
    sink = grad_sinks.get(w)
    if _is_native(rows):
        if sink is not None:
            _grouped(2, rows, dy, None, sink, g_start, g_len, E, N, K, accumulate=True)
            return None
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        _grouped(2, rows, dy, None, dw, g_start, g_len, E, N, K, accumulate=False)
        return dw.to(w.dtype)
    dw = torch.zeros(w.shape, dtype=torch.float32)
    for g, a, b in _grouped_ref_segments(g_start, g_len):
        dw[g % E] += dy[a:b].float().t() @ rows[a:b].float()
    if sink is not None:
        sink.add_(dw)
        return None
    return dw.to(w.dtype)


def _glinear_setup(ctx, inputs, output):
    rows, w, g_start, g_len = inputs
    ctx.save_for_backward(rows, w, g_start, g_len)


def _glinear_backward(ctx, dy):
    rows, w, g_start, g_len = ctx.saved_tensors
    E, N, K = w.shape
    dyc = dy.contiguous()
    if (core._GEMM_FORK and ctx.needs_input_grad[0] and ctx.needs_input_grad[1] and wgrad_store.active is None
            and _is_native(rows) and grad_sinks.get(w) is not None):
        # same fork as in the dense linear backward: the weight-gradient GEMM runs on a side stream
        cur = torch.cuda.current_stream(rows.device)
        side = core._side_stream(cur)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            _grouped_wgrad(rows, dyc, w, g_start, g_len)
        drows = torch.empty_like(rows, memory_format=torch.contiguous_format)
        _grouped(1, None, dyc, w, drows, g_start, g_len, E, N, K)
        if core._GEMM_FORK == 2 and core.deferred_join.depth > 0:
            for t in (rows, dyc, g_start, g_len):
                t.record_stream(side)
            core.deferred_join.pending[(cur.device.index, cur.cuda_stream)] = (cur, side)
        else:
            cur.wait_stream(side)
        return drows, None, None, None
    drows = None
    if ctx.needs_input_grad[0]:
        if _is_native(rows):
            drows = torch.empty_like(rows, memory_format=torch.contiguous_format)
            _grouped(1, None, dyc, w, drows, g_start, g_len, E, N, K)
        else:
            drows = torch.zeros_like(rows)
            for g, a, b in _grouped_ref_segments(g_start, g_len):
                drows[a:b] = dyc[a:b] @ w[g % E]
    dw = None
    if ctx.needs_input_grad[1]:
        if wgrad_store.active is not None:
            rd, dd = rows.detach(), dyc.detach()
            wgrad_store.active.append((lambda: _grouped_wgrad(rd, dd, w, g_start, g_len), w))
        else:
            dw = _grouped_wgrad(rows, dyc, w, g_start, g_len)
    return drows, dw, None, None


grouped_linear.register_autograd(_glinear_backward, setup_context=_glinear_setup)


# ----------------------------------------------------------------- combine
@torch.library.custom_op("piper::moe_combine", mutates_args=())
def moe_combine(rows: Tensor, pos: Tensor, weights: Tensor, g_start: Tensor, g_len: Tensor, counts: Tensor) -> Tensor:
    """out[t] = sum_j weights[t, j] * rows[pos[t*k + j]]."""
    T, k = weights.shape
    D = rows.shape[1]
    if _is_native(rows):
        _require_bf16(rows)
        out = torch.empty((T, D), dtype=rows.dtype, device=rows.device)
        native.lib().moe_combine(rows.contiguous(), pos, weights.contiguous(), out)
        return out
    picked = rows[pos.long()].float().reshape(T, k, D)
    return (picked * weights.float().unsqueeze(-1)).sum(1).to(rows.dtype)


@moe_combine.register_fake
def _(rows, pos, weights, g_start, g_len, counts):
    return rows.new_empty((weights.shape[0], rows.shape[1]))


def _combine_setup(ctx, inputs, output):
    rows, pos, weights, g_start, g_len, counts = inputs
    ctx.save_for_backward(rows, pos, weights, g_start, g_len, counts)


def _combine_backward(ctx, dout):
    rows, pos, weights, g_start, g_len, counts = ctx.saved_tensors
    T, k = weights.shape
    D = rows.shape[1]
    if _is_native(rows):
        drows = torch.empty_like(rows, memory_format=torch.contiguous_format)
        dweights = torch.empty_like(weights, memory_format=torch.contiguous_format)
        native.lib().moe_combine_bwd(rows.contiguous(), dout.contiguous(), pos, weights.contiguous(), drows, dweights,
                                     g_start, g_len, counts)
        return drows, None, dweights, None, None, None
    drows = torch.zeros_like(rows)
    g = dout.float().unsqueeze(1) * weights.float().unsqueeze(-1)
    drows[pos.long()] = g.reshape(T * k, D).to(rows.dtype)
    dweights = (rows[pos.long()].float().reshape(T, k, D) * dout.float().unsqueeze(1)).sum(-1)
    return drows, None, dweights.to(weights.dtype), None, None, None


moe_combine.register_autograd(_combine_backward, setup_context=_combine_setup)
