"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean():
    from piper_b200.ops import native

    yield
    native.check_status()


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _max_err(a, b):
    """Largest elementwise error, relative to the largest reference magnitude: one wrong element shows here even
    where the norm-wise error of a large tensor hides it."""
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def _close(a, b, tol):
    """Norm-wise relative error below ``tol`` and every element within ``4 * tol`` of the reference's scale."""
    assert a.shape == b.shape, (a.shape, b.shape)
    assert torch.isfinite(a.float()).all()
    return _rel_err(a, b) < tol and _max_err(a, b) < 4 * tol


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 192), (200, 328, 136), (4096, 1024, 512)])
def test_gemm_forward_layout(M, N, K):
    from piper_b200.ops import native

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    native.lib().gemm(a, b, c, False, False, False, native.status_tensor())
    ref = a.float() @ b.float().t()
    assert _close(c, ref, 1e-2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 320), (200, 328, 136)])
def test_gemm_dgrad_and_wgrad_layouts(M, N, K):
    from piper_b200.ops import native

    torch.manual_seed(1)
    st = native.status_tensor()
    # dgrad: C[M,N] = A[M,K] * Bs[K,N]  (B stored [K, N])
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    bs = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    native.lib().gemm(a, bs, c, False, True, False, st)
    assert _close(c, a.float() @ bs.float(), 1e-2)
    # wgrad: C[M,N] = As[K,M]^T * Bs[K,N], fp32 accumulate into an existing buffer
    as_ = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    ref = acc + as_.float().t() @ bs.float()
    native.lib().gemm(as_, bs, acc, True, True, True, st)
    assert _close(acc, ref, 1e-2)
    # A MN-major with B K-major
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c2 = torch.empty(M, N, device="cuda", dtype=torch.float32)
    native.lib().gemm(as_, b, c2, True, False, False, st)
    assert _close(c2, as_.float().t() @ b.float().t(), 1e-2)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (200, 328, 136), (2304, 4608, 192)])
def test_gemm_256_tile_all_layouts(M, N, K):
    """The 256x256-tile kernel against fp32 references: every operand layout, both epilogues, ragged edges and
    (last shape) more tiles than SMs so that CTAs walk several tiles and reuse their accumulator halves."""
    from piper_b200.ops import native

    torch.manual_seed(3)
    st = native.status_tensor()
    lib = native.lib()
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    at, bt = a.t().contiguous(), b.t().contiguous()          # [K, M], [K, N]
    ref = a.float() @ b.float().t()
    for a_op, a_mn in ((a, False), (at, True)):
        for b_op, b_mn in ((b, False), (bt, True)):
            c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            lib.gemm_tiled(a_op, b_op, c, a_mn, b_mn, False, st, 256)
            assert _close(c, ref, 1e-2), (a_mn, b_mn)
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    want = acc + ref
    lib.gemm_tiled(at, bt, acc, True, True, True, st, 256)
    assert _close(acc, want, 1e-2)
    c128 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    c256 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    lib.gemm_tiled(a, b, c128, False, False, False, st, 128)
    lib.gemm_tiled(a, b, c256, False, False, False, st, 256)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.equal(c128, c256)      # same k order and fp32 accumulation: identical bits


def test_linear_op_autograd():
    from piper_b200 import ops

    torch.manual_seed(2)
    x = torch.randn(2, 256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(768, 512, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_(True)
    y = ops.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert _close(y, yr, 1e-2)
    assert _close(x.grad, xr.grad, 1e-2)
    assert _close(w.grad, wr.grad, 1e-2)


@pytest.mark.parametrize("T,D", [(300, 256), (300, 2048), (1000, 4096), (300, 8192), (7, 4096)])
def test_rmsnorm_and_residual(T, D):
    from piper_b200 import ops

    torch.manual_seed(3)
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y, h = ops.add_rmsnorm(x, r, w, 1e-6)
    gy, gh = torch.randn_like(y), torch.randn_like(h)
    torch.autograd.backward([y, h], [gy, gh])
    xr, rr, wr = (t.detach().float().requires_grad_(True) for t in (x, r, w))
    hr = (xr + rr).to(torch.bfloat16).float() + 0 * (xr + rr)
    hr = xr + rr
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    torch.autograd.backward([yr, hr], [gy.float(), gh.float()])
    assert _close(y, yr, 1e-2) and _close(h, hr, 1e-2)
    assert _close(x.grad, xr.grad, 2e-2) and _close(r.grad, rr.grad, 2e-2)
    assert _close(w.grad, wr.grad, 2e-2)
    y2 = ops.rmsnorm(x.detach(), w.detach(), 1e-6)
    x0 = x.detach().float()
    assert _close(y2, x0 * torch.rsqrt(x0.pow(2).mean(-1, keepdim=True) + 1e-6) * w.detach().float(), 1e-2)


@pytest.mark.parametrize("hd,inter,qknorm,seqs", [(128, True, False, 2), (128, False, True, 2), (64, False, False, 2),
                                                  (64, True, True, 2), (128, False, True, 640), (64, True, True, 1200)])
def test_qk_rope(hd, inter, qknorm, seqs):
    """The large cases use 12 heads (two head chunks per token, the second one partial) and more tokens than one
    pass of the grid covers."""
    from piper_b200 import ops
    from piper_b200.ops.core import _qk_rope_ref

    torch.manual_seed(4)
    S, Hq, Hkv = (64, 4, 2) if seqs == 2 else (64, 8, 2)
    cos, sin = ops.rope_tables(hd, S, 10000.0, device="cuda")
    qkv = torch.randn(seqs * S, (Hq + 2 * Hkv) * hd, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    qw = torch.randn(hd, device="cuda", dtype=torch.bfloat16, requires_grad=True) if qknorm else None
    kw = torch.randn(hd, device="cuda", dtype=torch.bfloat16, requires_grad=True) if qknorm else None
    out = ops.qk_rope(qkv, cos, sin, qw, kw, S, Hq, Hkv, hd, inter, 1e-6)
    g = torch.randn_like(out)
    out.backward(g)
    q2 = qkv.detach().float().requires_grad_(True)
    qw2 = qw.detach().float().requires_grad_(True) if qknorm else None
    kw2 = kw.detach().float().requires_grad_(True) if qknorm else None
    ref = _qk_rope_ref(q2, cos, sin, qw2, kw2, S, Hq, Hkv, hd, inter, 1e-6)
    ref.backward(g.float())
    assert _close(out, ref, 1e-2)
    assert _close(qkv.grad, q2.grad, 2e-2)
    if qknorm:
        assert _close(qw.grad, qw2.grad, 3e-2) and _close(kw.grad, kw2.grad, 3e-2)


@pytest.mark.parametrize("B,S,Hq,Hkv,hd", [(1, 128, 2, 1, 128), (2, 256, 4, 2, 128), (1, 512, 4, 4, 64), (1, 1024, 8, 2, 128),
                                           (1, 4096, 32, 8, 128)])
def test_attention_fwd_bwd(B, S, Hq, Hkv, hd):
    from piper_b200 import ops
    from piper_b200.ops.core import _attention_ref

    torch.manual_seed(5)
    qkv = (torch.randn(B * S, (Hq + 2 * Hkv) * hd, device="cuda", dtype=torch.bfloat16)).requires_grad_(True)
    out = ops.attention(qkv, B, S, Hq, Hkv, hd)
    g = torch.randn_like(out)
    out.backward(g)
    q2 = qkv.detach().float().requires_grad_(True)
    ref, _ = _attention_ref(q2, B, S, Hq, Hkv, hd, 1.0 / math.sqrt(hd))
    ref.backward(g.float())
    assert _close(out, ref, 2e-2)
    W = (Hq + 2 * Hkv) * hd
    gq, gr = qkv.grad.view(-1, W), q2.grad.view(-1, W)
    assert _close(gq[:, : Hq * hd], gr[:, : Hq * hd], 3e-2)          # dQ
    assert _close(gq[:, Hq * hd: (Hq + Hkv) * hd], gr[:, Hq * hd: (Hq + Hkv) * hd], 3e-2)   # dK
    assert _close(gq[:, (Hq + Hkv) * hd:], gr[:, (Hq + Hkv) * hd:], 3e-2)   # dV


@pytest.mark.parametrize("T,F", [(9000, 776), (5000, 14336)])
def test_swiglu_grid_stride_walk(T, F):
    """More vectors than the grid has threads, with a row length that the grid stride does not divide."""
    from piper_b200 import ops

    torch.manual_seed(16)
    h = torch.randn(T, 2 * F, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    a = ops.swiglu(h)
    g = torch.randn_like(a)
    a.backward(g)
    hr = h.detach().float().requires_grad_(True)
    ar = torch.nn.functional.silu(hr[:, :F]) * hr[:, F:]
    ar.backward(g.float())
    assert _close(a, ar, 1e-2) and _close(h.grad, hr.grad, 1e-2)


def test_swiglu_embedding_ce_adam():
    from piper_b200 import ops
    from piper_b200.ops import native

    torch.manual_seed(6)
    h = torch.randn(333, 2 * 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    a = ops.swiglu(h)
    g = torch.randn_like(a)
    a.backward(g)
    hr = h.detach().float().requires_grad_(True)
    ar = torch.nn.functional.silu(hr[:, :1024]) * hr[:, 1024:]
    ar.backward(g.float())
    assert _close(a, ar, 1e-2) and _close(h.grad, hr.grad, 1e-2)

    table = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    tok = torch.randint(0, 1000, (4, 77), device="cuda")
    e = ops.embedding(tok, table)
    ge = torch.randn_like(e)
    e.backward(ge)
    tr = table.detach().float().requires_grad_(True)
    torch.nn.functional.embedding(tok, tr).backward(ge.float())
    assert torch.equal(e, table.detach()[tok])
    assert _close(table.grad, tr.grad, 1e-2)

    V = 5000
    logits = (torch.randn(257, V, device="cuda", dtype=torch.bfloat16) * 3).requires_grad_(True)
    labels = torch.randint(0, V, (257,), device="cuda")
    labels[5] = -100
    loss = ops.cross_entropy(logits, labels)
    loss.backward()
    lr = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, labels)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-3 * max(1.0, abs(ref.item()))
    assert _close(logits.grad, lr.grad, 2e-2)

    n = 100_003
    master = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    grad = torch.randn(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr = master.clone().requires_grad_(True)
    opt = torch.optim.Adam([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for step in (1, 2):
        native.lib().adam_flat(master, m, v, grad, p16, 1e-2, 0.9, 0.95, 1e-8, 0.0, step, 1.0, True)
        pr.grad = grad.clone()
        opt.step()
    assert _close(master, pr.detach(), 1e-5)
    assert _close(p16, pr.detach(), 1e-2)
