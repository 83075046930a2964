"""End-to-end equivalence on CPU/gloo: every parallel layout reproduces the single-process loss and gradients."""
import pytest
import torch

from tests.dist_utils import run_ranks

SEQ = 128


def _data(cfg, batch, seed=0):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, cfg.vocab_size, (batch, SEQ + 1), generator=g)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def _reference(batch, steps=1, lr=1e-3):
    from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.runtime.storage import materialize_module

    cfg = LLAMA_CONFIGS["tiny"]
    x, y = _data(cfg, batch)
    m = Transformer(cfg, SEQ, 1)
    m.load_const_attrs()
    materialize_module(m)
    opt = torch.optim.Adam(m.parameters(), lr=lr)
    out = {}
    for step in range(steps):
        opt.zero_grad()
        loss = cross_entropy_loss(m(x), y)
        loss.backward()
        if step == 0:
            out["loss"] = float(loss.detach())
            out["grads"] = {n: p.grad.clone() for n, p in m.named_parameters()}
        opt.step()
    out["params"] = {n: p.detach().clone() for n, p in m.named_parameters()}
    return out


def _worker(rank, world, schedule, num_stages, global_batch, dp, steps, ckpt=False):
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.runtime.layout import make_layout
    from piper_b200.compiler.schedule import stage_device_map

    cfg = LLAMA_CONFIGS["tiny"]
    x, y = _data(cfg, global_batch)
    layout = make_layout(stage_device_map(schedule), rank, world)
    per = global_batch // dp
    xs, ys = x[layout.dp_rank * per:(layout.dp_rank + 1) * per], y[layout.dp_rank * per:(layout.dp_rank + 1) * per]
    actor = piper_setup(Transformer, (cfg, SEQ, num_stages), optim_fn=torch.optim.Adam, example_inputs=[xs],
                        example_outputs=ys, model_dtype=torch.float32, const_attrs=Transformer.const_attrs(cfg, SEQ),
                        schedule_directives=schedule, device="cpu", activation_checkpointing=ckpt)
    actor.debug_keep_grads = True
    first = None
    for _ in range(steps):
        losses = piper_exec_dag(cross_entropy_loss)
        if first is None:
            first = ([float(l) for l in losses], dict(actor.last_grads))
    params = {k: v.detach().clone() for k, v in actor.named_parameters().items()}
    return {"losses": first[0], "grads": first[1], "params": params, "dp_rank": layout.dp_rank,
            "bucket_keys": list(actor.buckets)}


def _check(results, ref, dp, atol=1e-5, check_params=False):
    losses = [l for r in results for l in r["losses"]]
    assert losses, "no rank reported a loss"
    assert abs(sum(losses) / len(losses) - ref["loss"]) < atol
    seen = set()
    for r in results:
        for k, g in r["grads"].items():
            if isinstance(g, tuple):      # ZeRO shard: (offset inside the parameter, flat values)
                off, vals = g
                want = ref["grads"][k].reshape(-1)[off:off + vals.numel()]
                assert torch.allclose(vals, want, atol=atol), k
            else:
                assert torch.allclose(g, ref["grads"][k], atol=atol), k
            seen.add(k)
    assert seen == set(ref["grads"]), sorted(set(ref["grads"]) - seen)
    if check_params:
        for r in results:
            for k, p in r["params"].items():
                # Adam turns a 1e-8 gradient difference on a near-zero gradient into an lr-sized step
                # difference, so the bound is per-step lr for the maximum and tight for the mean
                d = (p - ref["params"][k]).abs()
                assert d.max() <= 2.5e-3 and d.mean() < 2e-5, (k, float(d.max()), float(d.mean()))


def _sched(places, mbs, extra=(), order=()):
    s = [{"op": "place", "filter": {"PP": i}, "devices": d, "stream": "pp_stream"} for i, d in enumerate(places)]
    s += list(extra)
    s.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": mbs})
    s += list(order)
    return s


def test_pp2_1f1b_matches_single_process(tmp_path):
    """Two annotate('PP') regions of two layers on two ranks, 1F1B over 4 microbatches of a batch of 8."""
    from piper_b200.compiler.builders import build_1f1b_schedule

    sched = _sched([[0], [1]], 4, order=build_1f1b_schedule(2, 4))
    res = run_ranks(2, _worker, (sched, 2, 8, 1, 1), tmp_path)
    _check(res, _reference(8), dp=1)


def test_pp2_zerobubble_with_activation_checkpointing(tmp_path):
    """Forward keeps segment inputs only; backward (here the split BWD_I/BWD_W form) recomputes the segment."""
    from piper_b200.compiler.builders import build_zerobubble_schedule

    sched = _sched([[0], [1]], 4, order=build_zerobubble_schedule(2, 4))
    res = run_ranks(2, _worker, (sched, 2, 8, 1, 1, True), tmp_path)
    _check(res, _reference(8), dp=1)


def test_dp2_allreduce_matches_single_process(tmp_path):
    sched = _sched([[0, 1]], 2, extra=[{"op": "replicate", "filter": {"PP": 0}, "devices": [0, 1],
                                        "reduce_stream": "dp_stream"}])
    res = run_ranks(2, _worker, (sched, 1, 8, 2, 2), tmp_path)
    _check(res, _reference(8, steps=2), dp=2, check_params=True)


@pytest.mark.parametrize("flags", [{"shard_grads": True}, {"shard_grads": True, "shard_params": True}])
def test_dp2_zero_matches_single_process(tmp_path, flags):
    sched = _sched([[0, 1]], 2, extra=[{"op": "replicate", "filter": {"PP": 0}, "devices": [0, 1],
                                        "gather_stream": "dp_stream", "reduce_stream": "dp_stream", **flags}])
    res = run_ranks(2, _worker, (sched, 1, 8, 2, 2), tmp_path)
    _check(res, _reference(8, steps=2), dp=2, check_params=True)


@pytest.mark.parametrize("flags", [{}, {"shard_grads": True, "shard_params": True}])
def test_pp2_dp2_1f1b_with_parameter_buckets_matches_single_process(tmp_path, flags):
    """Pipeline messages meet bucket chains: ``replicate.bucket_size`` splits each stage into per-bucket nodes, so
    sends leave from the last bucket of a chain and receives feed the first (plain and ZeRO-3 buckets)."""
    from piper_b200.compiler.builders import build_1f1b_schedule

    extra = [{"op": "replicate", "filter": {"PP": i}, "devices": d, "reduce_stream": "dp_stream",
              "gather_stream": "gather_stream", "bucket_size": 1, **flags} for i, d in enumerate([[0, 2], [1, 3]])]
    sched = _sched([[0, 2], [1, 3]], 2, extra=extra, order=build_1f1b_schedule(2, 2))
    res = run_ranks(4, _worker, (sched, 2, 8, 2, 2), tmp_path, timeout=600)
    assert any("bucket" in k for r in res for k in r.get("bucket_keys", []))
    _check(res, _reference(8, steps=2), dp=2, check_params=True)


def test_pp2_dp2_zerobubble_matches_single_process(tmp_path):
    from piper_b200.compiler.builders import build_zerobubble_schedule

    extra = [{"op": "replicate", "filter": {"PP": 0}, "devices": [0, 2], "reduce_stream": "dp_stream"},
             {"op": "replicate", "filter": {"PP": 1}, "devices": [1, 3], "reduce_stream": "dp_stream"}]
    sched = _sched([[0, 2], [1, 3]], 2, extra=extra, order=build_zerobubble_schedule(2, 2))
    res = run_ranks(4, _worker, (sched, 2, 8, 2, 1), tmp_path)
    _check(res, _reference(8), dp=2)


def test_interleaved_v_placement_four_stages_on_two_ranks(tmp_path):
    from piper_b200.compiler.builders import build_dualpipev_schedule

    sched = _sched([[0], [1], [1], [0]], 4, order=build_dualpipev_schedule(2, 4))
    res = run_ranks(2, _worker, (sched, 4, 8, 1, 1), tmp_path)
    _check(res, _reference(8), dp=1)


def _moe_reference(batch):
    from piper_b200.models.qwen3 import QWEN3_CONFIGS, PiperQwen3Model
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.runtime.storage import materialize_module

    cfg = QWEN3_CONFIGS["9M"]
    x, y = _data(cfg, batch)
    m = PiperQwen3Model(cfg, 1, SEQ)
    m.load_const_attrs()
    materialize_module(m)
    loss = cross_entropy_loss(m(x), y)
    loss.backward()
    return {"loss": float(loss.detach()), "grads": {n: p.grad.clone() for n, p in m.named_parameters()}}


def _moe_worker(rank, world, schedule, num_stages, global_batch, dp):
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.compiler.schedule import stage_device_map
    from piper_b200.models.qwen3 import QWEN3_CONFIGS, PiperQwen3Model
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.runtime.layout import make_layout

    cfg = QWEN3_CONFIGS["9M"]
    x, y = _data(cfg, global_batch)
    layout = make_layout(stage_device_map(schedule), rank, world)
    per = global_batch // dp
    xs, ys = x[layout.dp_rank * per:(layout.dp_rank + 1) * per], y[layout.dp_rank * per:(layout.dp_rank + 1) * per]
    actor = piper_setup(PiperQwen3Model, (cfg, num_stages, SEQ), optim_fn=torch.optim.Adam, example_inputs=[xs],
                        example_outputs=ys, model_dtype=torch.float32,
                        const_attrs=PiperQwen3Model.const_attrs(cfg, SEQ), schedule_directives=schedule, device="cpu")
    actor.debug_keep_grads = True
    losses = [float(l) for l in piper_exec_dag(cross_entropy_loss)]
    return {"losses": losses, "grads": dict(actor.last_grads), "dp_rank": layout.dp_rank}


def test_expert_parallel_dp2_ep2_matches_single_process(tmp_path):
    """True expert parallelism: experts partitioned over two ranks, rows exchanged with per-expert counts."""
    extra = [{"op": "replicate", "filter": {"PP": 0}, "devices": [0, 1], "reduce_stream": "dp_stream"},
             {"op": "shard", "filter": {"PP": 0, "EP": "*"}, "devices": [0, 1], "stream": "ep_stream"}]
    sched = _sched([[0, 1]], 2, extra=extra)
    res = run_ranks(2, _moe_worker, (sched, 1, 4, 2), tmp_path)
    ref = _moe_reference(4)
    losses = [l for r in res for l in r["losses"]]
    assert abs(sum(losses) / len(losses) - ref["loss"]) < 1e-5
    for r in res:
        for k, g in r["grads"].items():
            want = ref["grads"][k]
            if g.shape != want.shape:            # expert weights: this rank holds its slice of the experts
                per = want.shape[0] // 2
                want = want[r["dp_rank"] * per:(r["dp_rank"] + 1) * per]
            assert torch.allclose(g, want, atol=2e-5), (k, float((g - want).abs().max()))


def test_expert_groups_nested_in_data_parallel_sum_replica_gradients(tmp_path):
    """DP4 with two expert-parallel groups of two ranks: ranks 0 and 2 (1 and 3) hold the same experts, so their
    gradients are summed across the groups; every gradient equals the single-process one."""
    extra = [{"op": "replicate", "filter": {"PP": 0}, "devices": [0, 1, 2, 3], "reduce_stream": "dp_stream"},
             {"op": "shard", "filter": {"PP": 0, "EP": "*"}, "devices": [[0, 1], [2, 3]], "stream": "ep_stream"}]
    sched = _sched([[0, 1, 2, 3]], 1, extra=extra)
    res = run_ranks(4, _moe_worker, (sched, 1, 4, 4), tmp_path, timeout=600)
    ref = _moe_reference(4)
    losses = [l for r in res for l in r["losses"]]
    assert abs(sum(losses) / len(losses) - ref["loss"]) < 1e-5
    sliced = 0
    for r in res:
        for k, g in r["grads"].items():
            want = ref["grads"][k]
            if g.shape != want.shape:
                per = want.shape[0] // 2
                i = r["dp_rank"] % 2                      # position inside the expert-parallel group
                want = want[i * per:(i + 1) * per]
                sliced += 1
            assert torch.allclose(g, want, atol=2e-5), (k, r["dp_rank"], float((g - want).abs().max()))
    assert sliced > 0


def _row_gather_worker(rank, world):
    import torch.distributed as dist

    from piper_b200.runtime.storage import AdamConfig, ParamSlot, ParamStorage

    dist.init_process_group("gloo", rank=rank, world_size=world)
    shapes = {"a.weight": (300, 16), "norm.weight": (130,), "b.weight": (64, 24)}
    slots = [ParamSlot(pos=i, fqn=k, shape=v, dtype=torch.float32, requires_grad=True)
             for i, (k, v) in enumerate(shapes.items())]
    st = ParamStorage("bucket", slots, torch.device("cpu"), torch.float32, "zero3", rank, world, dist.group.WORLD,
                      AdamConfig())
    st.all_gather_params()
    before = st.flat_params.clone()
    st.convert_to_rows(lambda name, n, dt: torch.zeros(n, dtype=dt))
    st.param_users = 1
    st.free_params()
    assert not st.params_live
    st.all_gather_params()                   # outside a step: rebuilt from every rank's row pieces
    same = bool(torch.equal(st.flat_params, before))
    full = st.full_param_tensor()
    dist.destroy_process_group()
    return same and bool(torch.equal(full, before))


def test_row_sharded_bucket_regathers_its_parameters_outside_a_step(tmp_path):
    assert all(run_ranks(2, _row_gather_worker, (), tmp_path))
