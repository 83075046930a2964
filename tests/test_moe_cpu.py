"""MoE ops on CPU: reference bodies and autograd formulas against a dense formulation."""
import pytest
import torch

from piper_b200.ops import moe as M


def _dense_moe(x, gate_w, w13, w2, k):
    p = torch.softmax(x @ gate_w.t(), dim=-1)
    w, idx = torch.topk(p, k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    out = torch.zeros_like(x)
    F = w13.shape[1] // 2
    for t in range(x.shape[0]):
        for j in range(k):
            e = int(idx[t, j])
            h = w13[e] @ x[t]
            a = torch.nn.functional.silu(h[:F]) * h[F:]
            out[t] += w[t, j] * (w2[e] @ a)
    return out


def test_moe_pipeline_matches_dense_formulation_with_grads():
    torch.manual_seed(0)
    T, D, E, k, F = 24, 16, 4, 2, 8
    x = torch.randn(T, D, requires_grad=True)
    gate_w = torch.randn(E, D, requires_grad=True)
    w13 = (torch.randn(E, 2 * F, D) * 0.3).requires_grad_(True)
    w2 = (torch.randn(E, D, F) * 0.3).requires_grad_(True)
    from piper_b200 import ops

    weights, idx, counts = M.moe_route(ops.linear(x, gate_w), k, True)
    assert int(counts.sum()) == T * k
    rows, pos, g_start, g_len, _ = M.moe_dispatch(x, idx, counts)
    assert (g_len % 128 == 0).all() and len(set(pos.tolist())) == T * k
    gs, gl = M.moe_group_table(counts, w13)
    assert torch.equal(gs, g_start) and torch.equal(gl, g_len)
    h = M.grouped_linear(rows, w13, gs, gl)
    o = M.grouped_linear(ops.swiglu(h), w2, gs, gl)
    out = M.moe_combine(o, pos, weights, g_start, g_len, counts)
    g = torch.randn_like(out)
    out.backward(g)

    xr, gr, w13r, w2r = (t.detach().clone().requires_grad_(True) for t in (x, gate_w, w13, w2))
    ref = _dense_moe(xr, gr, w13r, w2r, k)
    ref.backward(g)
    assert torch.allclose(out, ref, atol=1e-5)
    for a, b in ((x, xr), (gate_w, gr), (w13, w13r), (w2, w2r)):
        assert torch.allclose(a.grad, b.grad, atol=1e-4), (a.grad - b.grad).abs().max()


def test_qwen3_model_traces_into_pp_and_ep_segments():
    from piper_b200.api import _reset_annotation_state, compile_training_dags
    from piper_b200.models.qwen3 import QWEN3_CONFIGS, PiperQwen3Model

    cfg = QWEN3_CONFIGS["9M"]
    got = {}

    def backend(gm, example_inputs):
        got["gm"] = gm
        return gm.forward

    _reset_annotation_state()
    torch._dynamo.reset()
    with torch.device("meta"):
        model = PiperQwen3Model(cfg, 2, 128)
    with torch.no_grad():
        torch.compile(model, backend=backend, fullgraph=True)(torch.empty(2, 128, dtype=torch.long, device="meta"))
    directives = [
        {"op": "place", "filter": {"PP": 0}, "devices": [0, 2], "stream": "pp_stream"},
        {"op": "place", "filter": {"PP": 1}, "devices": [1, 3], "stream": "pp_stream"},
        {"op": "replicate", "filter": {"PP": 0}, "devices": [0, 2], "reduce_stream": "dp_stream"},
        {"op": "replicate", "filter": {"PP": 1}, "devices": [1, 3], "reduce_stream": "dp_stream"},
        {"op": "shard", "filter": {"PP": 0, "EP": "*"}, "devices": [0, 2], "stream": "ep_stream"},
        {"op": "shard", "filter": {"PP": 1, "EP": "*"}, "devices": [1, 3], "stream": "ep_stream"},
        {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2},
    ]
    dag, per_dev, segs = compile_training_dags(got["gm"], directives)
    tags = [s.tag for s in segs]
    assert tags[0] == {"PP": 0} and tags[1] == {"PP": 0, "EP": 0} and {"PP": 1, "EP": 2} in tags
    # the exchanged tensor is the routed row buffer (2-D, width = model dim), never the residual stream
    for s in segs[:-1]:
        if "EP" in s.a2a_boundary_after["to_tag"] and "EP" not in s.tag:
            i = s.a2a_boundary_after["tensor_idx"]
            outs = list(s.gm.graph.nodes)[-1].args[0]
            val = outs[i].meta["example_value"]
            assert val.dim() == 2 and val.shape[0] == M.row_capacity(2 * 128, cfg.top_k, cfg.num_experts)
            assert s.a2a_boundary_after["counts_idx"] is not None
    kinds = [n.node_kind for n in per_dev[0].nodes.values()]
    assert kinds.count("A2A_COMM") == 2 * 2 * 2 * 2      # 2 MoE layers x (in, out) x (fwd, bwd) x 2 microbatches
    ep_fwd = [n for n in per_dev[0].nodes.values() if n.node_kind == "COMPUTE" and "EP" in n.tag and n.compute_subkind == "FWD"]
    assert all(n.node_meta.get("ep_shard") for n in ep_fwd)
    assert not any(n.node_kind == "REDUCE_COMM" and "EP" in n.tag for n in per_dev[0].nodes.values())


@pytest.mark.parametrize("schedule", ["1f1b", "dualpipev", "zerobubble"])
def test_expert_exchange_buffer_plan_from_the_dispatch_order(schedule):
    """The slot planner of the peer-memory expert exchanges, on a CPU-compiled plan: every exchange has its four
    roles, exchanges whose lifetimes overlap in the dispatch order never share a slot or a gradient buffer, the
    slot count is the largest overlap, and every buffer is handed back by a node of this rank's own order."""
    from piper_b200 import piper_setup
    from piper_b200.compiler import builders
    from piper_b200.models.qwen3 import QWEN3_CONFIGS, PiperQwen3Model
    from piper_b200.parallel.ep_fused import FusedExpertRuntime, source_capacity

    cfg, seq, mbs = QWEN3_CONFIGS["9M"], 32, 4
    x = torch.randint(0, cfg.vocab_size, (mbs, seq))
    stages = 2 if schedule == "dualpipev" else 1
    sched = [{"op": "place", "filter": {"PP": s}, "devices": [0], "stream": "pp_stream"} for s in range(stages)]
    sched += [{"op": "shard", "filter": {"PP": s, "EP": "*"}, "devices": [0], "stream": "ep_stream"} for s in range(stages)]
    sched.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": mbs})
    sched += {"1f1b": builders.build_1f1b_schedule, "dualpipev": builders.build_dualpipev_schedule,
              "zerobubble": builders.build_zerobubble_schedule}[schedule](1, mbs)
    actor = piper_setup(PiperQwen3Model, (cfg, stages, seq), optim_fn=torch.optim.Adam, example_inputs=[x],
                        example_outputs=x, model_dtype=torch.float32,
                        const_attrs=PiperQwen3Model.const_attrs(cfg, seq), schedule_directives=sched, device="cpu")
    rt = FusedExpertRuntime(actor, [0], None, 1.0, 8, 1.25)
    layers = cfg.n_layers
    assert len(rt.exchanges) == mbs * layers
    roles = sorted(k for k, _ in rt.role.values())
    assert roles.count("F_in") == roles.count("F_out") == roles.count("B_in") == roles.count("B_out") == mbs * layers
    xs = list(rt.exchanges.values())
    if schedule != "dualpipev":                          # DualPipeV splits the backward of some microbatches only
        assert all(x.split_backward == (schedule == "zerobubble") for x in xs)
    peak = 0
    for i, a in enumerate(xs):
        assert 0 <= a.slot < rt.slots and a.first < a.last < len(actor.order)
        peak = max(peak, sum(1 for b in xs if b.first <= a.first <= b.last))
        for b in xs[i + 1:]:
            if not (a.last < b.first or b.last < a.first):
                assert a.slot != b.slot
            for span, buf in (("gin_span", "gin_buf"), ("gret_span", "gret_buf")):
                (a0, a1), (b0, b1) = getattr(a, span), getattr(b, span)
                if not (a1 < b0 or b1 < a0):
                    assert getattr(a, buf) != getattr(b, buf)
    assert rt.slots == peak                               # interval colouring is optimal
    freed = [act for acts in rt.after.values() for act, _ in acts]
    assert freed.count("free_recv") == freed.count("free_ret") == freed.count("free_gret") == mbs * layers
    assert set(rt.after) <= set(actor.order)
    # capacity: worst case without a factor, the balanced share plus padding reserve with one
    assert source_capacity(4096, 8, 32, 4, None) >= 4096 * 8
    assert source_capacity(4096, 8, 32, 4, 1.25) == (10240 + 32 * 127 + 127) // 128 * 128
