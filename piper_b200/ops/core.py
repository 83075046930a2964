"""``torch.ops.piper.*``: the traced compute ops of the bundled models.

Each op is a ``torch.library.custom_op`` so that TorchDynamo records it as a
single FX node (the graph splitter and the schedule see whole ops, never their
internals), with

* a CUDA body that calls the hand-written sm_100a kernels through
  ``torch.ops.piper_c`` (bf16 only; a missing native library is an error),
* a CPU body in plain PyTorch fp32/bf16 math, which is both the oracle of the
  numerics tests and what the CPU/gloo multi-process tests execute,
* a fake (meta) body for tracing on the ``meta`` device,
* an autograd formula whose backward again calls the kernels directly.

Two pieces of runtime state change what the linear op's backward does with
its weight gradient (the reference keeps per-parameter ``.grad`` tensors and
copies them into the ZeRO buffer afterwards, ``src/runtime.py:249-282``; here
the weight-gradient GEMM writes where the gradient finally lives):

* ``grad_sinks``: parameter storage address -> fp32 view of the flat gradient
  bucket.  If the weight has a sink, ``dW`` is accumulated into it by the GEMM
  epilogue and autograd sees no gradient for the weight.
* ``wgrad_store``: while a split backward (``BWD_I``) runs, the weight-gradient
  GEMMs are queued instead of executed; the matching ``BWD_W`` task drains the
  queue.  This is what makes zero-bubble schedules actually defer the wgrad
  work (the reference re-walks the autograd graph instead,
  ``src/executors.py:353-476``).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
from torch import Tensor

from . import native

# --------------------------------------------------------------------------
# runtime state consulted by backward formulas
# --------------------------------------------------------------------------


class GradSinks:
    """Maps a parameter's storage address to the fp32 buffer its gradient accumulates into."""

    def __init__(self) -> None:
        self._sinks: dict[int, Tensor] = {}

    def register(self, param: Tensor, sink: Tensor) -> None:
        assert sink.dtype == torch.float32 and sink.numel() == param.numel()
        self._sinks[param.data_ptr()] = sink.view(param.shape)

    def unregister(self, param: Tensor) -> None:
        self._sinks.pop(param.data_ptr(), None)

    def get(self, param: Tensor) -> Optional[Tensor]:
        return self._sinks.get(param.data_ptr())

    def clear(self) -> None:
        self._sinks.clear()


grad_sinks = GradSinks()


class WgradStore:
    """Queue of deferred weight-gradient GEMMs of one backward-input pass: (thunk returning dW or None, weight)."""

    def __init__(self) -> None:
        self.active: Optional[list] = None

    def begin(self) -> list:
        self.active = []
        return self.active

    def end(self) -> list:
        q, self.active = self.active, None
        return q or []

    @staticmethod
    def drain(queue: list) -> list[tuple[Tensor, Tensor]]:
        """Run the queued GEMMs.  Returns (weight, dW) pairs for weights without a sink."""
        out = []
        with torch.no_grad():
            for fn, w in queue:
                dw = fn()
                if dw is not None:
                    out.append((w, dw))
        queue.clear()
        return out


wgrad_store = WgradStore()

# ZeRO-3 with the fused lowering: weight address -> launcher of the GEMM that gathers that weight's rows from the
# data-parallel peers while it multiplies by them (registered by ``parallel/fused.py`` when the parameters of a
# segment are materialised, consumed by the first ``linear`` that uses the weight).
gather_gemms: dict = {}


def _is_native(t: Tensor) -> bool:
    return t.is_cuda


def _require_bf16(*ts: Tensor) -> None:
    for t in ts:
        if t.dtype != torch.bfloat16:
            raise TypeError(f"the sm_100a kernels take bfloat16 tensors, got {t.dtype}")


# --------------------------------------------------------------------------
# linear
# --------------------------------------------------------------------------


def _gemm(a: Tensor, b: Tensor, out: Tensor, a_mn: bool, b_mn: bool, accumulate: bool = False) -> Tensor:
    native.lib().gemm(a, b, out, a_mn, b_mn, accumulate, native.status_tensor(a.device))
    return out


@torch.library.custom_op("piper::linear", mutates_args=())
def linear(x: Tensor, w: Tensor) -> Tensor:
    """y[..., N] = x[..., K] @ w[N, K]^T."""
    if _is_native(x):
        _require_bf16(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = torch.empty((x2.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
        fused_gather = gather_gemms.pop(w.data_ptr(), None) if gather_gemms else None
        if fused_gather is not None:
            fused_gather(x2, y)
        else:
            _gemm(x2, w, y, False, False)
        return y.view(*x.shape[:-1], w.shape[0])
    return torch.nn.functional.linear(x, w)


@linear.register_fake
def _(x, w):
    return x.new_empty((*x.shape[:-1], w.shape[0]))


def _linear_dgrad(dy2: Tensor, w: Tensor) -> Tensor:
    if _is_native(dy2):
        dx = torch.empty((dy2.shape[0], w.shape[1]), dtype=dy2.dtype, device=dy2.device)
        # dX[T,K] = dY[T,N] * W[N,K]: B operand is W read as [contraction N][K contiguous].
        return _gemm(dy2, w, dx, False, True)
    return dy2 @ w


def _linear_wgrad(x2: Tensor, dy2: Tensor, w: Tensor) -> Optional[Tensor]:
    """dW[N,K] = dY^T X, into the weight's fp32 sink if it has one (returns None then)."""
    sink = grad_sinks.get(w)
    if _is_native(x2):
        if sink is not None:
            _gemm(dy2, x2, sink, True, True, accumulate=True)
            return None
        dw = torch.empty_like(w)
        return _gemm(dy2, x2, dw, True, True)
    dw = dy2.t() @ x2
    if sink is not None:
        sink.add_(dw.to(torch.float32))
        return None
    return dw.to(w.dtype)


# The input-gradient and weight-gradient GEMMs of one linear layer are independent.  Each is a persistent kernel
# with one CTA per SM whose last round of tiles leaves SMs idle (256 tiles on 148 SMs: 40 idle SMs in the second
# round); launched on two streams, the CTAs of the second kernel start on the SMs the first one has left.
# PIPER_GEMM_FORK=0 runs them one after the other on the current stream; 1 joins the side stream at the end of
# every linear backward; 2 (default) joins only when the enclosing ``deferred_join`` block ends (the executor
# wraps the backward pass of a segment in one), so a weight-gradient GEMM also runs under the kernels that follow
# it; outside such a block, and for weights without a gradient sink, 2 behaves like 1.  Measured on the 8B-shape
# step on one GPU: 3,227 ms (0), 3,180 ms (1), 3,066 ms (2), identical losses.
_GEMM_FORK = int(os.environ.get("PIPER_GEMM_FORK", "2") or 0)
_side_streams: dict = {}


class deferred_join:
    """Scope inside which forked weight-gradient GEMMs are joined once, at exit, instead of per layer."""

    depth = 0
    pending: dict = {}

    def __enter__(self):
        deferred_join.depth += 1
        return self

    def __exit__(self, *exc):
        deferred_join.depth -= 1
        if deferred_join.depth == 0:
            for cur, side in deferred_join.pending.values():
                cur.wait_stream(side)
            deferred_join.pending.clear()
        return False


def _side_stream(cur: "torch.cuda.Stream") -> "torch.cuda.Stream":
    key = (cur.device.index, cur.cuda_stream)
    side = _side_streams.get(key)
    if side is None:
        side = _side_streams[key] = torch.cuda.Stream(device=cur.device)
    return side


def _linear_setup(ctx, inputs, output):
    x, w = inputs
    ctx.save_for_backward(x, w)


def _linear_backward(ctx, dy):
    x, w = ctx.saved_tensors
    dy2 = dy.reshape(-1, dy.shape[-1])
    if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    deferred = wgrad_store.active is not None
    if (_GEMM_FORK and ctx.needs_input_grad[0] and ctx.needs_input_grad[1] and not deferred and _is_native(dy2)):
        cur = torch.cuda.current_stream(dy2.device)
        side = _side_stream(cur)
        dw_out = None if grad_sinks.get(w) is not None else torch.empty_like(w)   # allocated on the current stream
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            if dw_out is None:
                _linear_wgrad(x2, dy2, w)
            else:
                _gemm(dy2, x2, dw_out, True, True)
        dx = _linear_dgrad(dy2, w).view(x.shape)
        if _GEMM_FORK == 2 and deferred_join.depth > 0 and dw_out is None:
            # the operands may be freed before the side stream has read them: tell the allocator
            x2.record_stream(side)
            dy2.record_stream(side)
            deferred_join.pending[(cur.device.index, cur.cuda_stream)] = (cur, side)
        else:
            cur.wait_stream(side)   # everything later on this stream, frees of x and dy included, follows both GEMMs
        return dx, dw_out
    dx = None
    if ctx.needs_input_grad[0]:
        dx = _linear_dgrad(dy2, w).view(x.shape)
    dw = None
    if ctx.needs_input_grad[1]:
        if deferred:
            xd, dyd = x2.detach(), dy2.detach()
            wgrad_store.active.append((lambda: _linear_wgrad(xd, dyd, w), w))
        else:
            dw = _linear_wgrad(x2, dy2, w)
    return dx, dw


linear.register_autograd(_linear_backward, setup_context=_linear_setup)

# --------------------------------------------------------------------------
# RMSNorm (optionally fused with the residual add)
# --------------------------------------------------------------------------


@torch.library.custom_op("piper::rmsnorm_fwd", mutates_args=())
def rmsnorm_fwd(x: Tensor, w: Tensor, eps: float) -> tuple[Tensor, Tensor]:
    """Returns (y, rstd) with y = x * rsqrt(mean(x^2) + eps) * w computed in fp32."""
    if _is_native(x):
        _require_bf16(x, w)
        xc = x.contiguous()
        y = torch.empty_like(xc)
        rstd = torch.empty(xc.numel() // xc.shape[-1], dtype=torch.float32, device=x.device)
        native.lib().rmsnorm_fwd(xc, None, w, y, None, rstd, eps)
        return y, rstd
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    y = (xf * rstd.unsqueeze(-1) * w.float()).to(x.dtype)
    return y, rstd.reshape(-1)


@rmsnorm_fwd.register_fake
def _(x, w, eps):
    return torch.empty_like(x), x.new_empty((x.numel() // x.shape[-1],), dtype=torch.float32)


def _rmsnorm_bwd_impl(dy: Tensor, x: Tensor, w: Tensor, rstd: Tensor, dres: Optional[Tensor]):
    """Returns (dx, dw or None); dw goes to the weight's fp32 sink when it has one."""
    sink = grad_sinks.get(w)
    if _is_native(x):
        dyc = dy.contiguous()
        xc = x.contiguous()
        D = x.shape[-1]
        T = x.numel() // D
        dx = torch.empty_like(xc)
        nb = native.lib().rmsnorm_bwd_num_partials(T)
        partial = torch.empty((nb, D), dtype=torch.float32, device=x.device)
        if sink is not None:
            native.lib().rmsnorm_bwd(dyc, xc, w, rstd, dres, dx, partial, sink.view(-1), None, True)
            return dx, None
        dw = torch.empty_like(w)
        native.lib().rmsnorm_bwd(dyc, xc, w, rstd, dres, dx, partial, None, dw, False)
        return dx, dw
    xf, dyf, wf = x.float(), dy.float(), w.float()
    r = rstd.view(*x.shape[:-1], 1)
    xhat = xf * r
    g = dyf * wf
    dot = (g * xhat).mean(-1, keepdim=True)
    dx = r * (g - xhat * dot)
    if dres is not None:
        dx = dx + dres.float()
    dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0)
    if sink is not None:
        sink.add_(dw)
        return dx.to(x.dtype), None
    return dx.to(x.dtype), dw.to(w.dtype)


def _rmsnorm_setup(ctx, inputs, output):
    x, w, _eps = inputs
    _y, rstd = output
    ctx.save_for_backward(x, w, rstd)


def _rmsnorm_backward(ctx, dy, _drstd):
    x, w, rstd = ctx.saved_tensors
    dx, dw = _rmsnorm_bwd_impl(dy, x, w, rstd, None)
    return dx, dw, None


rmsnorm_fwd.register_autograd(_rmsnorm_backward, setup_context=_rmsnorm_setup)


def rmsnorm(x: Tensor, w: Tensor, eps: float = 1e-6) -> Tensor:
    return rmsnorm_fwd(x, w, eps)[0]


@torch.library.custom_op("piper::add_rmsnorm_fwd", mutates_args=())
def add_rmsnorm_fwd(x: Tensor, res: Tensor, w: Tensor, eps: float) -> tuple[Tensor, Tensor, Tensor]:
    """h = x + res; y = rmsnorm(h) * w.  Returns (y, h, rstd)."""
    if _is_native(x):
        _require_bf16(x, res, w)
        xc, rc = x.contiguous(), res.contiguous()
        y = torch.empty_like(xc)
        h = torch.empty_like(xc)
        rstd = torch.empty(xc.numel() // xc.shape[-1], dtype=torch.float32, device=x.device)
        native.lib().rmsnorm_fwd(xc, rc, w, y, h, rstd, eps)
        return y, h, rstd
    h = (x.float() + res.float()).to(x.dtype)
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps)
    y = (hf * rstd.unsqueeze(-1) * w.float()).to(x.dtype)
    return y, h, rstd.reshape(-1)


@add_rmsnorm_fwd.register_fake
def _(x, res, w, eps):
    return (torch.empty_like(x), torch.empty_like(x),
            x.new_empty((x.numel() // x.shape[-1],), dtype=torch.float32))


def _add_rmsnorm_setup(ctx, inputs, output):
    _x, _res, w, _eps = inputs
    _y, h, rstd = output
    ctx.save_for_backward(h, w, rstd)


def _add_rmsnorm_backward(ctx, dy, dh, _drstd):
    h, w, rstd = ctx.saved_tensors
    if dy is None:
        return dh, dh, None, None
    dres = None if dh is None else dh.contiguous()
    dx, dw = _rmsnorm_bwd_impl(dy, h, w, rstd, dres)
    return dx, dx, dw, None


add_rmsnorm_fwd.register_autograd(_add_rmsnorm_backward, setup_context=_add_rmsnorm_setup)


def add_rmsnorm(x: Tensor, res: Tensor, w: Tensor, eps: float = 1e-6) -> tuple[Tensor, Tensor]:
    """Returns (rmsnorm(x + res) * w, x + res)."""
    y, h, _ = add_rmsnorm_fwd(x, res, w, eps)
    return y, h


@torch.library.custom_op("piper::residual_add", mutates_args=())
def residual_add(a: Tensor, b: Tensor) -> Tensor:
    """a + b for two activations of the same shape (the residual add that is not fused into a norm)."""
    if _is_native(a) and a.dtype == torch.bfloat16 and a.numel() % 8 == 0:
        out = torch.empty_like(a, memory_format=torch.contiguous_format)
        native.lib().add_bf16(a.contiguous(), b.contiguous(), out)
        return out
    return a + b


@residual_add.register_fake
def _(a, b):
    return torch.empty_like(a)


residual_add.register_autograd(lambda ctx, g: (g, g))


# --------------------------------------------------------------------------
# QK-norm + RoPE on the packed qkv projection
# --------------------------------------------------------------------------


def rope_tables(head_dim: int, max_seq: int, theta: float, device=None) -> tuple[Tensor, Tensor]:
    """cos/sin tables [max_seq, head_dim/2] in fp32."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.outer(torch.arange(max_seq, dtype=torch.float32, device=device), inv)
    return torch.cos(ang), torch.sin(ang)


def _qk_rope_ref(qkv, cos, sin, qw, kw, S, Hq, Hkv, hd, interleaved, eps, sign=1.0):
    T = qkv.numel() // ((Hq + 2 * Hkv) * hd)
    x = qkv.reshape(T, Hq + 2 * Hkv, hd).float()
    q, k, v = x[:, :Hq], x[:, Hq:Hq + Hkv], x[:, Hq + Hkv:]

    def norm(t, w):
        if w is None:
            return t
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w.float()

    pos = torch.arange(T, device=qkv.device) % S
    c = cos[pos].unsqueeze(1).float()
    s = sin[pos].unsqueeze(1).float() * sign

    def rot(t):
        if interleaved:
            a, b = t[..., 0::2], t[..., 1::2]
            return torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2)
        a, b = t[..., : hd // 2], t[..., hd // 2:]
        return torch.cat((a * c - b * s, b * c + a * s), dim=-1)

    out = torch.cat((rot(norm(q, qw)), rot(norm(k, kw)), v), dim=1)
    return out.reshape(qkv.shape).to(qkv.dtype)


@torch.library.custom_op("piper::qk_rope", mutates_args=())
def qk_rope(qkv: Tensor, cos: Tensor, sin: Tensor, qw: Optional[Tensor], kw: Optional[Tensor], S: int,
            Hq: int, Hkv: int, hd: int, interleaved: bool, eps: float) -> Tensor:
    """Applies optional per-head RMSNorm and rotary embedding to the q and k heads of packed qkv."""
    if _is_native(qkv):
        _require_bf16(qkv)
        qc = qkv.contiguous()
        out = torch.empty_like(qc)
        native.lib().qk_rope_fwd(qc, out, cos, sin, qw, kw, S, Hq, Hkv, hd, interleaved, eps)
        return out
    return _qk_rope_ref(qkv, cos, sin, qw, kw, S, Hq, Hkv, hd, interleaved, eps)


@qk_rope.register_fake
def _(qkv, cos, sin, qw, kw, S, Hq, Hkv, hd, interleaved, eps):
    return torch.empty_like(qkv)


def _qk_rope_setup(ctx, inputs, output):
    qkv, cos, sin, qw, kw, S, Hq, Hkv, hd, interleaved, eps = inputs
    ctx.cfg = (S, Hq, Hkv, hd, interleaved, eps)
    ctx.has_w = (qw is not None, kw is not None)
    saved = [cos, sin]
    if qw is not None or kw is not None:
        saved.append(qkv)
    if qw is not None:
        saved.append(qw)
    if kw is not None:
        saved.append(kw)
    ctx.save_for_backward(*saved)


def _qk_rope_backward(ctx, dout):
    S, Hq, Hkv, hd, interleaved, eps = ctx.cfg
    saved = list(ctx.saved_tensors)
    cos, sin = saved[0], saved[1]
    rest = saved[2:]
    qkv = rest.pop(0) if any(ctx.has_w) else None
    qw = rest.pop(0) if ctx.has_w[0] else None
    kw = rest.pop(0) if ctx.has_w[1] else None
    dqw = dkw = None
    if _is_native(dout):
        dc = dout.contiguous()
        din = torch.empty_like(dc)
        sq = grad_sinks.get(qw) if qw is not None else None
        sk = grad_sinks.get(kw) if kw is not None else None
        bq = sq.view(-1) if sq is not None else (torch.zeros(hd, dtype=torch.float32, device=dout.device) if qw is not None else None)
        bk = sk.view(-1) if sk is not None else (torch.zeros(hd, dtype=torch.float32, device=dout.device) if kw is not None else None)
        native.lib().qk_rope_bwd(dc, qkv if qkv is not None else dc, din, cos, sin, qw, kw, bq, bk, S, Hq, Hkv,
                                 hd, interleaved, eps)
        if qw is not None and sq is None:
            dqw = bq.to(qw.dtype)
        if kw is not None and sk is None:
            dkw = bk.to(kw.dtype)
    else:
        if qkv is None:
            din = _qk_rope_ref(dout, cos, sin, None, None, S, Hq, Hkv, hd, interleaved, eps, sign=-1.0)
        else:
            with torch.enable_grad():
                qin = qkv.detach().float().requires_grad_(True)
                qwf = qw.detach().float().requires_grad_(True) if qw is not None else None
                kwf = kw.detach().float().requires_grad_(True) if kw is not None else None
                o = _qk_rope_ref(qin, cos, sin, qwf, kwf, S, Hq, Hkv, hd, interleaved, eps)
                wrt = [qin] + [t for t in (qwf, kwf) if t is not None]
                grads = list(torch.autograd.grad(o, wrt, dout.float()))
            din = grads.pop(0).to(dout.dtype)
            for name, wt in (("q", qw), ("k", kw)):
                if wt is None:
                    continue
                gw = grads.pop(0)
                sink = grad_sinks.get(wt)
                if sink is not None:
                    sink.add_(gw.view(sink.shape))
                elif name == "q":
                    dqw = gw.to(wt.dtype)
                else:
                    dkw = gw.to(wt.dtype)
    return din, None, None, dqw, dkw, None, None, None, None, None, None


qk_rope.register_autograd(_qk_rope_backward, setup_context=_qk_rope_setup)

# --------------------------------------------------------------------------
# causal GQA attention on packed qkv
# --------------------------------------------------------------------------


def _attention_ref(qkv: Tensor, B: int, S: int, Hq: int, Hkv: int, hd: int, scale: float):
    x = qkv.reshape(B, S, Hq + 2 * Hkv, hd).float()
    q = x[:, :, :Hq].transpose(1, 2)
    k = x[:, :, Hq:Hq + Hkv].transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    v = x[:, :, Hq + Hkv:].transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    s = (q @ k.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.softmax(s, dim=-1) @ v
    return o.transpose(1, 2).reshape(B * S, Hq * hd), lse


@torch.library.custom_op("piper::attention_fwd", mutates_args=())
def attention_fwd(qkv: Tensor, B: int, S: int, Hq: int, Hkv: int, hd: int, scale: float) -> tuple[Tensor, Tensor]:
    """Causal grouped-query attention.  qkv: [B*S, (Hq+2Hkv)*hd] -> (out [B*S, Hq*hd], lse [B,Hq,S])."""
    if _is_native(qkv):
        _require_bf16(qkv)
        qc = qkv.contiguous()
        out = torch.empty((B * S, Hq * hd), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=qkv.device)
        native.lib().attn_fwd(qc, out, lse, B, S, Hq, Hkv, hd, scale, native.status_tensor(qkv.device))
        return out, lse
    o, lse = _attention_ref(qkv, B, S, Hq, Hkv, hd, scale)
    return o.to(qkv.dtype), lse


@attention_fwd.register_fake
def _(qkv, B, S, Hq, Hkv, hd, scale):
    return qkv.new_empty((B * S, Hq * hd)), qkv.new_empty((B, Hq, S), dtype=torch.float32)


def _attention_setup(ctx, inputs, output):
    qkv, B, S, Hq, Hkv, hd, scale = inputs
    out, lse = output
    ctx.cfg = (B, S, Hq, Hkv, hd, scale)
    ctx.save_for_backward(qkv, out, lse)


def _attention_backward(ctx, dout, _dlse):
    B, S, Hq, Hkv, hd, scale = ctx.cfg
    qkv, out, lse = ctx.saved_tensors
    if _is_native(qkv):
        qc = qkv.contiguous()
        dqkv = torch.empty_like(qc)
        delta = torch.empty((B, Hq, S), dtype=torch.float32, device=qkv.device)
        native.lib().attn_bwd(qc, out, dout.contiguous(), lse, delta, dqkv, B, S, Hq, Hkv, hd, scale,
                              native.status_tensor(qkv.device))
        return dqkv.view(qkv.shape), None, None, None, None, None, None
    with torch.enable_grad():
        qin = qkv.detach().float().requires_grad_(True)
        o, _ = _attention_ref(qin, B, S, Hq, Hkv, hd, scale)
        (g,) = torch.autograd.grad(o, qin, dout.float())
    return g.to(qkv.dtype), None, None, None, None, None, None


attention_fwd.register_autograd(_attention_backward, setup_context=_attention_setup)


def attention(qkv: Tensor, B: int, S: int, Hq: int, Hkv: int, hd: int, scale: Optional[float] = None) -> Tensor:
    return attention_fwd(qkv, B, S, Hq, Hkv, hd, 1.0 / math.sqrt(hd) if scale is None else scale)[0]


# --------------------------------------------------------------------------
# SwiGLU
# --------------------------------------------------------------------------


@torch.library.custom_op("piper::swiglu", mutates_args=())
def swiglu(h13: Tensor) -> Tensor:
    """act = silu(h13[..., :F]) * h13[..., F:]."""
    F = h13.shape[-1] // 2
    if _is_native(h13):
        _require_bf16(h13)
        hc = h13.contiguous()
        act = torch.empty((*h13.shape[:-1], F), dtype=h13.dtype, device=h13.device)
        native.lib().swiglu_fwd(hc, act)
        return act
    g, u = h13[..., :F].float(), h13[..., F:].float()
    return (torch.nn.functional.silu(g) * u).to(h13.dtype)


@swiglu.register_fake
def _(h13):
    return h13.new_empty((*h13.shape[:-1], h13.shape[-1] // 2))


def _swiglu_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0])


def _swiglu_backward(ctx, dact):
    (h13,) = ctx.saved_tensors
    if _is_native(h13):
        d = torch.empty_like(h13, memory_format=torch.contiguous_format)
        native.lib().swiglu_bwd(h13.contiguous(), dact.contiguous(), d)
        return d
    F = h13.shape[-1] // 2
    g, u, da = h13[..., :F].float(), h13[..., F:].float(), dact.float()
    sg = torch.sigmoid(g)
    dg = da * u * sg * (1 + g * (1 - sg))
    du = da * g * sg
    return torch.cat((dg, du), dim=-1).to(h13.dtype)


swiglu.register_autograd(_swiglu_backward, setup_context=_swiglu_setup)

# --------------------------------------------------------------------------
# embedding
# --------------------------------------------------------------------------


@torch.library.custom_op("piper::embedding", mutates_args=())
def embedding(tokens: Tensor, table: Tensor) -> Tensor:
    if _is_native(table):
        _require_bf16(table)
        out = torch.empty((*tokens.shape, table.shape[1]), dtype=table.dtype, device=table.device)
        native.lib().embedding_fwd(tokens.contiguous(), table, out, native.status_tensor(table.device))
        return out
    return torch.nn.functional.embedding(tokens, table)


@embedding.register_fake
def _(tokens, table):
    return table.new_empty((*tokens.shape, table.shape[1]))


def _embedding_setup(ctx, inputs, output):
    tokens, table = inputs
    ctx.save_for_backward(tokens, table)


def _embedding_backward(ctx, dout):
    tokens, table = ctx.saved_tensors
    sink = grad_sinks.get(table)
    if _is_native(table):
        buf = sink if sink is not None else torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        native.lib().embedding_bwd(tokens.contiguous(), dout.contiguous(), buf)
        return None, (None if sink is not None else buf.to(table.dtype))
    g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
    g.index_add_(0, tokens.reshape(-1), dout.reshape(-1, table.shape[1]).float())
    if sink is not None:
        sink.add_(g)
        return None, None
    return None, g.to(table.dtype)


embedding.register_autograd(_embedding_backward, setup_context=_embedding_setup)

# --------------------------------------------------------------------------
# cross-entropy (per-token losses)
# --------------------------------------------------------------------------


@torch.library.custom_op("piper::cross_entropy_fwd", mutates_args=())
def cross_entropy_fwd(logits: Tensor, labels: Tensor, ignore_index: int) -> tuple[Tensor, Tensor]:
    """Per-token loss [T] (fp32) and log-sum-exp [T] of logits [T, V]."""
    if _is_native(logits):
        _require_bf16(logits)
        lg = logits if logits.stride(-1) == 1 and logits.stride(0) % 8 == 0 else logits.contiguous()
        T = lg.shape[0]
        loss = torch.empty(T, dtype=torch.float32, device=lg.device)
        lse = torch.empty(T, dtype=torch.float32, device=lg.device)
        native.lib().ce_fwd(lg, labels.contiguous(), loss, lse, ignore_index)
        return loss, lse
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    loss = torch.nn.functional.cross_entropy(lf, labels, ignore_index=ignore_index, reduction="none")
    return loss, lse


@cross_entropy_fwd.register_fake
def _(logits, labels, ignore_index):
    T = logits.shape[0]
    return logits.new_empty((T,), dtype=torch.float32), logits.new_empty((T,), dtype=torch.float32)


def _ce_setup(ctx, inputs, output):
    logits, labels, ignore_index = inputs
    _loss, lse = output
    ctx.ignore_index = ignore_index
    ctx.save_for_backward(logits, labels, lse)


def _ce_backward(ctx, dloss, _dlse):
    logits, labels, lse = ctx.saved_tensors
    if _is_native(logits):
        # The kernel takes one scalar scale; per-token upstream gradients other
        # than a broadcast scalar take the PyTorch expression below.
        d = dloss if dloss.stride(0) == 0 or dloss.numel() == 1 else None
        if d is not None:
            gs = d.reshape(-1)[:1].to(torch.float32).contiguous()
            lg = logits if logits.stride(-1) == 1 and logits.stride(0) % 8 == 0 else logits.contiguous()
            out = torch.empty_like(lg)
            native.lib().ce_bwd(lg, labels.contiguous(), lse, gs, 1.0, out, ctx.ignore_index)
            return out, None, None
    p = torch.exp(logits.float() - lse.unsqueeze(-1))
    valid = labels != ctx.ignore_index
    idx = labels.clamp(min=0).unsqueeze(-1)
    p.scatter_add_(1, idx, -torch.ones_like(idx, dtype=p.dtype))
    p = p * (dloss.float() * valid.float()).unsqueeze(-1)
    return p.to(logits.dtype), None, None


cross_entropy_fwd.register_autograd(_ce_backward, setup_context=_ce_setup)


def cross_entropy(logits: Tensor, labels: Tensor, ignore_index: int = -100, reduction: str = "mean") -> Tensor:
    """Cross-entropy over [.., V] logits without materialising fp32 probabilities."""
    lg = logits.reshape(-1, logits.shape[-1])
    lb = labels.reshape(-1)
    loss, _ = cross_entropy_fwd(lg, lb, ignore_index)
    if reduction == "none":
        return loss
    if reduction == "sum":
        return loss.sum()
    n = (lb != ignore_index).sum().clamp(min=1)
    return loss.sum() / n
