"""CPU checks of the custom ops' reference bodies and autograd formulas against plain PyTorch."""
import math

import torch

from piper_b200 import ops


def test_linear_matches_torch_and_grads():
    torch.manual_seed(0)
    x = torch.randn(3, 5, 8, requires_grad=True)
    w = torch.randn(6, 8, requires_grad=True)
    y = ops.linear(x, w)
    ref = torch.nn.functional.linear(x.detach(), w.detach())
    assert torch.allclose(y, ref, atol=1e-6)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().clone().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    torch.nn.functional.linear(xr, wr).backward(g)
    assert torch.allclose(x.grad, xr.grad, atol=1e-5)
    assert torch.allclose(w.grad, wr.grad, atol=1e-5)


def test_linear_grad_sink_and_deferred_wgrad():
    torch.manual_seed(0)
    x = torch.randn(4, 8, requires_grad=True)
    w = torch.randn(6, 8, requires_grad=True)
    sink = torch.zeros(6, 8)
    ops.grad_sinks.register(w, sink)
    try:
        q = ops.wgrad_store.begin()
        y = ops.linear(x, w)
        g = torch.randn_like(y)
        y.backward(g)
        ops.wgrad_store.end()
        assert w.grad is None and sink.abs().sum() == 0 and len(q) == 1
        ops.wgrad_store.drain(q)
        assert torch.allclose(sink, g.t() @ x.detach(), atol=1e-5)
    finally:
        ops.grad_sinks.clear()


def test_rmsnorm_and_add_rmsnorm_grads():
    torch.manual_seed(0)
    x = torch.randn(2, 4, 16, requires_grad=True)
    r = torch.randn(2, 4, 16, requires_grad=True)
    w = torch.randn(16, requires_grad=True)
    y, h = ops.add_rmsnorm(x, r, w, 1e-6)
    (y.sum() + (h * h).sum()).backward()
    xr, rr, wr = (t.detach().clone().requires_grad_(True) for t in (x, r, w))
    hr = xr + rr
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    (yr.sum() + (hr * hr).sum()).backward()
    assert torch.allclose(y, yr, atol=1e-5)
    assert torch.allclose(x.grad, xr.grad, atol=1e-4)
    assert torch.allclose(r.grad, rr.grad, atol=1e-4)
    assert torch.allclose(w.grad, wr.grad, atol=1e-4)


def test_attention_matches_sdpa():
    torch.manual_seed(0)
    B, S, Hq, Hkv, hd = 2, 16, 4, 2, 8
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * hd, requires_grad=True)
    out = ops.attention(qkv, B, S, Hq, Hkv, hd)
    x = qkv.detach().reshape(B, S, Hq + 2 * Hkv, hd)
    q = x[:, :, :Hq].transpose(1, 2)
    k = x[:, :, Hq:Hq + Hkv].transpose(1, 2).repeat_interleave(2, 1)
    v = x[:, :, Hq + Hkv:].transpose(1, 2).repeat_interleave(2, 1)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert torch.allclose(out, ref.transpose(1, 2).reshape(B * S, Hq * hd), atol=1e-5)
    out.sum().backward()
    assert qkv.grad is not None and torch.isfinite(qkv.grad).all()


def test_qk_rope_is_orthogonal_and_backward_matches_autograd():
    torch.manual_seed(0)
    S, Hq, Hkv, hd = 8, 2, 1, 8
    cos, sin = ops.rope_tables(hd, S, 10000.0)
    qkv = torch.randn(2 * S, (Hq + 2 * Hkv) * hd, requires_grad=True)
    for inter in (True, False):
        out = ops.qk_rope(qkv, cos, sin, None, None, S, Hq, Hkv, hd, inter, 1e-6)
        assert torch.allclose(out.pow(2).sum(), qkv.pow(2).sum(), rtol=1e-5)
        g = torch.randn_like(out)
        (gin,) = torch.autograd.grad(out, qkv, g)
        from piper_b200.ops.core import _qk_rope_ref
        q2 = qkv.detach().clone().requires_grad_(True)
        (gref,) = torch.autograd.grad(_qk_rope_ref(q2, cos, sin, None, None, S, Hq, Hkv, hd, inter, 1e-6), q2, g)
        assert torch.allclose(gin, gref, atol=1e-5)


def test_swiglu_embedding_cross_entropy():
    torch.manual_seed(0)
    h = torch.randn(5, 12, requires_grad=True)
    a = ops.swiglu(h)
    hr = h.detach().clone().requires_grad_(True)
    ar = torch.nn.functional.silu(hr[:, :6]) * hr[:, 6:]
    assert torch.allclose(a, ar, atol=1e-6)
    g = torch.randn_like(a)
    a.backward(g)
    ar.backward(g)
    assert torch.allclose(h.grad, hr.grad, atol=1e-5)

    table = torch.randn(10, 4, requires_grad=True)
    tok = torch.tensor([[1, 2, 2], [0, 9, 1]])
    e = ops.embedding(tok, table)
    e.sum().backward()
    tr = table.detach().clone().requires_grad_(True)
    torch.nn.functional.embedding(tok, tr).sum().backward()
    assert torch.allclose(table.grad, tr.grad)

    logits = torch.randn(7, 11, requires_grad=True)
    labels = torch.randint(0, 11, (7,))
    labels[3] = -100
    loss = ops.cross_entropy(logits, labels)
    lr = logits.detach().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, labels)
    assert torch.allclose(loss, ref, atol=1e-6)
    loss.backward()
    ref.backward()
    assert torch.allclose(logits.grad, lr.grad, atol=1e-6)
