"""MoE kernels on the GPU against the PyTorch fp32 reference bodies of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("T,E,k", [(300, 8, 2), (1024, 128, 8)])
def test_router_forward_backward(T, E, k):
    from piper_b200.ops import moe as M, native

    torch.manual_seed(0)
    logits = (torch.randn(T, E, device="cuda") * 2).to(torch.bfloat16).requires_grad_(True)
    w, idx, counts = M.moe_route(logits, k, True)
    lr = logits.detach().cpu().float().requires_grad_(True)
    p = torch.softmax(lr, dim=-1)
    # bf16 logits tie often and tie-breaking is implementation-defined: check the selection by value
    kth = torch.topk(p, k, dim=-1).values[:, -1:]
    sel = torch.gather(p, 1, idx.cpu().long())
    assert (sel >= kth - 1e-6).all()
    assert all(len(set(r)) == k for r in idx.cpu().tolist())
    assert torch.equal(counts.cpu(), torch.bincount(idx.cpu().reshape(-1).long(), minlength=E).to(torch.int32))
    wr = sel / sel.sum(-1, keepdim=True)
    assert _rel(w, wr) < 1e-3
    g = torch.randn(T, k, device="cuda")
    (w * g).sum().backward()
    (wr * g.cpu()).sum().backward()
    assert _rel(logits.grad, lr.grad) < 2e-2
    native.check_status()


@pytest.mark.parametrize("T,D,E,k,F", [(256, 256, 8, 2, 128), (512, 512, 16, 4, 256), (1000, 2048, 128, 8, 768)])
def test_dispatch_grouped_mlp_combine(T, D, E, k, F):
    from piper_b200 import ops
    from piper_b200.ops import moe as M, native

    torch.manual_seed(1)
    x = (torch.randn(T, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    logits = torch.randn(T, E, device="cuda").to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * F, D, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    w2 = (torch.randn(E, D, F, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    weights, idx, counts = M.moe_route(logits, k, True)
    weights = weights.detach().requires_grad_(True)
    rows, pos, g_start, g_len, epc = M.moe_dispatch(x, idx, counts)
    gs, gl = M.moe_group_table(epc, w13)
    h = M.grouped_linear(rows, w13, gs, gl)
    o = M.grouped_linear(ops.swiglu(h), w2, gs, gl)
    out = M.moe_combine(o, pos, weights, g_start, g_len, counts)
    g = torch.randn_like(out)
    out.backward(g)
    native.check_status()

    # the same pipeline with the reference bodies on the CPU in fp32, reusing the GPU's routing decisions
    xr = x.detach().cpu().float().requires_grad_(True)
    w13r = w13.detach().cpu().float().requires_grad_(True)
    w2r = w2.detach().cpu().float().requires_grad_(True)
    wr = weights.detach().cpu().requires_grad_(True)
    rows_r, pos_r, gs_r, gl_r, _ = M.moe_dispatch(xr, idx.cpu(), counts.cpu())
    h_r = M.grouped_linear(rows_r, w13r, gs_r, gl_r)
    o_r = M.grouped_linear(ops.swiglu(h_r), w2r, gs_r, gl_r)
    out_r = M.moe_combine(o_r, pos_r, wr, gs_r, gl_r, counts.cpu())
    out_r.backward(g.cpu().float())
    assert torch.equal(gs.cpu(), gs_r) and torch.equal(gl.cpu(), gl_r)
    assert sorted(pos.tolist()) == sorted(pos_r.tolist())
    assert _rel(out, out_r) < 2e-2
    assert _rel(x.grad, xr.grad) < 3e-2
    assert _rel(weights.grad, wr.grad) < 3e-2
    assert _rel(w13.grad, w13r.grad) < 3e-2
    assert _rel(w2.grad, w2r.grad) < 3e-2


def test_qwen3_moe_model_trains_on_one_gpu():
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.models.qwen3 import PiperQwen3Model, Qwen3Config
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.ops import native

    cfg = Qwen3Config(dim=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128, vocab_size=2048, num_experts=16,
                      top_k=4, moe_hidden=256, max_seq_len=256)
    seq = 256
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, cfg.vocab_size, (4, seq + 1), generator=g)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0]},
             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2}]
    piper_setup(PiperQwen3Model, (cfg, 1, seq), optim_fn=torch.optim.Adam, optim_kwargs={"lr": 1e-3},
                example_inputs=[x], example_outputs=y, model_dtype=torch.bfloat16,
                const_attrs=PiperQwen3Model.const_attrs(cfg, seq), schedule_directives=sched, device="cuda")
    first = [float(v) for v in piper_exec_dag(cross_entropy_loss)]
    for _ in range(8):
        last = [float(v) for v in piper_exec_dag(cross_entropy_loss)]
    native.check_status()
    assert all(v == v for v in first + last)
    assert sum(last) < sum(first) - 0.5, (first, last)


def test_grouped_gemm_with_no_rows():
    """A rank that receives no rows in an expert exchange: forward/input-gradient products are empty and the
    weight gradient is zero (or left untouched when accumulating)."""
    from piper_b200.ops import native

    dev = torch.device("cuda")
    E, N, K = 4, 256, 128
    lib, st = native.lib(), native.status_tensor(dev)
    w = torch.randn(E, N, K, device=dev, dtype=torch.bfloat16)
    rows = torch.empty(0, K, device=dev, dtype=torch.bfloat16)
    dy = torch.empty(0, N, device=dev, dtype=torch.bfloat16)
    g_start = torch.zeros(2 * E, dtype=torch.int32, device=dev)
    g_len = torch.zeros(2 * E, dtype=torch.int32, device=dev)
    out = torch.empty(0, N, device=dev, dtype=torch.bfloat16)
    lib.grouped_gemm(0, rows, None, w, out, g_start, g_len, E, N, K, False, st)
    dx = torch.empty(0, K, device=dev, dtype=torch.bfloat16)
    lib.grouped_gemm(1, None, dy, w, dx, g_start, g_len, E, N, K, False, st)
    dw = torch.full((E, N, K), 3.0, device=dev)
    lib.grouped_gemm(2, rows, dy, None, dw, g_start, g_len, E, N, K, True, st)
    assert torch.all(dw == 3.0)
    lib.grouped_gemm(2, rows, dy, None, dw, g_start, g_len, E, N, K, False, st)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.all(dw == 0.0)


@pytest.mark.parametrize("sources,E,N,K", [(3, 4, 512, 192), (2, 8, 320, 256)])
def test_grouped_gemm_with_groups_from_several_sources(sources, E, N, K):
    """Rows grouped by (source, local expert) with gaps between the sources' regions, empty groups and ragged
    output widths: forward, input gradient and weight gradient against per-segment fp32 products."""
    from piper_b200.ops import native

    torch.manual_seed(3)
    dev = torch.device("cuda")
    lib, st = native.lib(), native.status_tensor(dev)
    blocks = torch.randint(0, 4, (sources * E,)).tolist()          # 128-row blocks per group, some empty
    blocks[1] = 0
    region = (sum(blocks) // sources + 3) * 128                     # every source's region, with slack
    g_start, g_len, at = [], [], 0
    for s in range(sources):
        at = max(at, s * region)
        for e in range(E):
            n = blocks[s * E + e] * 128
            g_start.append(at)
            g_len.append(n)
            at += n
    R = at + 128
    gs = torch.tensor(g_start, dtype=torch.int32, device=dev)
    gl = torch.tensor(g_len, dtype=torch.int32, device=dev)
    w = (torch.randn(E, N, K, device=dev) * 0.1).to(torch.bfloat16)
    rows = torch.randn(R, K, device=dev).to(torch.bfloat16)
    dy = torch.randn(R, N, device=dev).to(torch.bfloat16)
    out = torch.zeros(R, N, device=dev, dtype=torch.bfloat16)
    dx = torch.zeros(R, K, device=dev, dtype=torch.bfloat16)
    dw = torch.zeros(E, N, K, device=dev)
    lib.grouped_gemm(0, rows, None, w, out, gs, gl, E, N, K, False, st)
    lib.grouped_gemm(1, None, dy, w, dx, gs, gl, E, N, K, False, st)
    lib.grouped_gemm(2, rows, dy, None, dw, gs, gl, E, N, K, False, st)
    torch.cuda.synchronize()
    native.check_status()
    want_dw = torch.zeros_like(dw)
    for g, (a, n) in enumerate(zip(g_start, g_len)):
        if n == 0:
            continue
        e = g % E
        ref = rows[a:a + n].float() @ w[e].float().t()
        assert (out[a:a + n].float() - ref).abs().max() <= 2e-2 * ref.abs().max(), g
        ref = dy[a:a + n].float() @ w[e].float()
        assert (dx[a:a + n].float() - ref).abs().max() <= 2e-2 * ref.abs().max(), g
        want_dw[e] += dy[a:a + n].float().t() @ rows[a:a + n].float()
    assert (dw - want_dw).abs().max() <= 2e-2 * want_dw.abs().max()
    assert torch.count_nonzero(out[R - 128:]) == 0                  # rows outside every group are not written
