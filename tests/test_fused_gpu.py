"""Fused compute+collective kernels: bounded peer wait (1 GPU) and equivalence with the NCCL lowering (2 GPUs)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_wait_times_out_cleanly():
    """A peer flag that nothing sets: the wait kernel gives up after the deadline, reports status 2 with the tag of
    the wait, the reduction kernel behind it does nothing, and the context stays usable."""
    from piper_b200.ops import native

    lib = native.lib()
    dev = torch.device("cuda")
    flags = torch.zeros(6, device=dev, dtype=torch.int64)
    abort = torch.zeros(1, dtype=torch.int32, device=dev)
    status = native.status_tensor()
    status.zero_()
    lib.ep_wait(flags, 0, 2, 1, 0.2, status, 11, abort)          # waits for two peers to reach use 1
    n = 4096
    grads = [torch.ones(n, device=dev), torch.ones(n, device=dev)]
    ptr = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    master = torch.zeros(n // 2, device=dev)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    shard = torch.zeros(n // 2, device=dev, dtype=torch.bfloat16)
    table = torch.tensor([[0], [0], [n // 2], [n]], dtype=torch.int64, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    lib.zero_reduce(ptr(grads), None, master, m, v, shard, None, table, 0, 2, False, True, 1e-3, 0.9, 0.999, 1e-8,
                    0.0, False, 1, 1.0, ptr([flags, flags]), 2, 1, counter, abort, 8)
    torch.cuda.synchronize()
    assert int(abort.item()) == 1
    with pytest.raises(native.PiperCommTimeout) as err:
        native.check_status()
    assert "[11," in str(err.value)
    assert int(status.item()) == 0          # reset by check_status
    assert torch.equal(master, torch.zeros_like(master))   # nothing was updated
    x = torch.ones(8, device=dev) * 2       # the context still works
    assert float(x.sum()) == 16.0


@pytest.mark.parametrize("dp", [2, 4, 3])
def test_zero_reduce_and_gather_kernels_with_emulated_ranks(dp):
    """The reduce-scatter + Adam kernel and the gather kernel, one launch per emulated rank with every rank's
    buffers in this GPU's memory (no launch waits for another), against the plain formulas."""
    from piper_b200.ops import native
    from piper_b200.runtime.storage import ALIGN, ParamSlot, ParamStorage

    lib = native.lib()
    dev = torch.device("cuda")
    torch.manual_seed(dp)
    shapes = [(300, 64), (130,), (64, 128), (1000, 8)]
    slots, off = [], 0
    for i, sh in enumerate(shapes):
        n = 1
        for d in sh:
            n *= d
        slots.append(ParamSlot(pos=i, fqn=f"p{i}", shape=sh, dtype=torch.bfloat16, requires_grad=True, offset=off, numel=n))
        off += (n + ALIGN - 1) // ALIGN * ALIGN
    numel = (off + ALIGN * dp - 1) // (ALIGN * dp) * (ALIGN * dp)
    table_py, S = ParamStorage.row_layout(slots, dp)
    table = torch.tensor([[s.offset for s in slots], [t[0] for t in table_py], [t[1] for t in table_py],
                          [(s.numel + 63) // 64 * 64 for s in slots]], dtype=torch.int64, device=dev)
    ptr = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    valid = torch.zeros(numel, dtype=torch.bool, device=dev)
    for s in slots:
        valid[s.offset:s.offset + s.numel] = True
    params0 = (torch.randn(numel, device=dev) * 0.1 * valid).to(torch.bfloat16)
    grads = [torch.randn(numel, device=dev) * valid for _ in range(dp)]
    grads2 = [torch.randn(numel, device=dev) * valid for _ in range(dp)]
    gsum = sum(grads) + sum(grads2)
    full_grads = [g.clone() for g in grads]
    full_params = [params0.clone() for _ in range(dp)]
    flags = [torch.zeros(3 * dp, dtype=torch.int64, device=dev) for _ in range(dp)]
    abort = torch.zeros(1, dtype=torch.int32, device=dev)
    st = {}

    def pieces(r):
        for s, (sh, stride) in zip(slots, table_py):
            a = s.offset + r * stride
            e = min(s.offset + s.numel, a + stride)
            if a < e:
                yield a, e, sh

    for r in range(dp):
        master = torch.zeros(S, device=dev)
        shard_p = torch.zeros(S, device=dev, dtype=torch.bfloat16)
        for a, e, sh in pieces(r):
            master[sh:sh + e - a] = params0[a:e].float()
            shard_p[sh:sh + e - a] = params0[a:e]
        st[r] = dict(master=master, m=torch.zeros(S, device=dev), v=torch.zeros(S, device=dev), shard_p=shard_p,
                     shard_g=torch.zeros(S, device=dev), counter=torch.zeros(1, dtype=torch.int32, device=dev))
    lr, b1, b2, eps, wd, scale = 1e-2, 0.9, 0.95, 1e-8, 0.1, 0.25

    def launch(r, final):
        d = st[r]
        lib.zero_reduce(ptr(full_grads), d["shard_g"], d["master"], d["m"], d["v"], d["shard_p"],
                        ptr(full_params) if final else None, table, r, dp, True, final, lr, b1, b2, eps, wd, True, 1,
                        scale, ptr(flags), dp, 1 + int(final), d["counter"], abort, 16)

    for r in range(dp):                       # first gradient chain: accumulate only
        launch(r, False)
    torch.cuda.synchronize()
    for r in range(dp):
        for a, e, sh in pieces(r):
            want = sum(g[a:e] for g in grads)
            assert torch.allclose(st[r]["shard_g"][sh:sh + e - a], want, atol=1e-5)
            assert torch.count_nonzero(full_grads[r][a:e]) == 0          # own piece cleared
    for r in range(dp):                       # second chain: new gradients everywhere, then the final reduction
        full_grads[r].copy_(grads2[r])
    for r in range(dp):
        launch(r, True)
    torch.cuda.synchronize()
    native.check_status()
    g = gsum * scale
    m_ref = (1 - b1) * g
    v_ref = (1 - b2) * g * g
    w0 = params0.float()
    w_ref = w0 - lr * (m_ref / (1 - b1)) / ((v_ref / (1 - b2)).sqrt() + eps) - lr * wd * w0
    for r in range(dp):
        assert all(int(f[dp + r]) == 2 for f in flags)                   # DONE published to every rank
        for a, e, sh in pieces(r):
            assert torch.allclose(st[r]["master"][sh:sh + e - a], w_ref[a:e], atol=1e-5, rtol=1e-5)
            assert torch.count_nonzero(st[r]["shard_g"][sh:sh + e - a]) == 0
            new16 = st[r]["master"][sh:sh + e - a].to(torch.bfloat16)
            assert torch.equal(st[r]["shard_p"][sh:sh + e - a], new16)
            for q in range(dp):                                            # update stored into every rank's buffer
                assert torch.equal(full_params[q][a:e], new16)
    # gather: every rank's shard back into a full buffer, with and without a skipped parameter
    shards = [st[r]["shard_p"] for r in range(dp)]
    full = torch.zeros(numel, device=dev, dtype=torch.bfloat16)
    lib.zero_gather(ptr(shards), full, table, dp, -1, -1, None, 16)
    torch.cuda.synchronize()
    for s in slots:
        assert torch.equal(full[s.offset:s.offset + s.numel], full_params[0][s.offset:s.offset + s.numel])
    full.zero_()
    lib.zero_gather(ptr(shards), full, table, dp, 0, -1, None, 16)
    torch.cuda.synchronize()
    assert torch.count_nonzero(full[:slots[0].numel]) == 0
    s = slots[2]
    assert torch.equal(full[s.offset:s.offset + s.numel], full_params[0][s.offset:s.offset + s.numel])
    lib.zero_gather(ptr(shards), full, table, dp, -1, 0, None, 16)       # then only the parameter left out
    torch.cuda.synchronize()
    assert torch.equal(full[:slots[0].numel], full_params[0][:slots[0].numel])


def _dp_worker(rank, world, fused, steps, mode="allreduce"):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["PIPER_FUSED"] = "1" if fused else "0"
    import torch
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.models.llama3 import LlamaConfig, Transformer
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.ops import native

    torch.cuda.set_device(rank)
    cfg = LlamaConfig(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=1024, ffn_hidden=512, max_seq_len=128)
    seq = 128
    g = torch.Generator().manual_seed(7)
    tok = torch.randint(0, cfg.vocab_size, (8, seq + 1), generator=g)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    per = 8 // world
    xs, ys = x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per]
    devs = list(range(world))
    rep = {"op": "replicate", "filter": {"PP": 0}, "devices": devs, "reduce_stream": "dp_stream"}
    if mode == "zero2":
        rep.update({"shard_grads": True, "bucket_size": 1})
    elif mode == "zero3":
        rep.update({"shard_params": True, "gather_stream": "gather_stream", "bucket_size": 1})
    elif mode == "bucketed":
        rep.update({"bucket_size": 1})
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": devs}, rep,
             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2}]
    actor = piper_setup(Transformer, (cfg, seq, 1), optim_fn=torch.optim.Adam, optim_kwargs={"lr": 1e-3},
                        example_inputs=[xs], example_outputs=ys, model_dtype=torch.bfloat16,
                        const_attrs=Transformer.const_attrs(cfg, seq), schedule_directives=sched, device="cuda")
    assert (actor.fused is not None) == fused
    losses = []
    for _ in range(steps):
        losses.append([float(v) for v in piper_exec_dag(cross_entropy_loss)])
    torch.cuda.synchronize()
    native.check_status()
    params = {k: v.float().cpu() for k, v in actor.named_parameters().items()}
    return {"losses": losses, "params": params, "buckets": len(actor.buckets),
            "gather_gemms": sum(1 for b in (actor.fused.buckets.values() if actor.fused else ()) if b.first_slot >= 0)}


def _dp_modes_worker(rank, world, modes, steps):
    """Every data-parallel mode with the fused and with the NCCL lowering, in one set of processes."""
    out = {}
    for mode in modes:
        for fused in (True, False):
            out[(mode, fused)] = _dp_worker(rank, world, fused, steps, mode)
    return out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_data_parallel_paths_match_the_nccl_lowering_on_two_gpus(tmp_path):
    from tests.dist_utils import run_ranks

    modes = ["allreduce", "bucketed", "zero2", "zero3"]
    res = run_ranks(2, _dp_modes_worker, (modes, 4), tmp_path, timeout=900)
    for mode in modes:
        fused = [r[(mode, True)] for r in res]
        base = [r[(mode, False)] for r in res]
        if mode != "allreduce":
            assert fused[0]["buckets"] > 1, mode
        if mode == "zero3":
            assert fused[0]["gather_gemms"] >= 1        # some bucket gathers its first weight inside the GEMM
        # replicas agree with each other bit-for-bit after the fused update
        for k in fused[0]["params"]:
            assert torch.equal(fused[0]["params"][k], fused[1]["params"][k]), (mode, k)
        # and with the NCCL lowering up to reduction order and bf16 rounding
        for k, p in fused[0]["params"].items():
            d = (p - base[0]["params"][k]).abs()
            assert d.max() <= 8e-3 and d.mean() < 2e-4, (mode, k, float(d.max()), float(d.mean()))
        assert abs(fused[0]["losses"][-1][0] - base[0]["losses"][-1][0]) < 5e-2, mode
        assert fused[0]["losses"][-1][0] < fused[0]["losses"][0][0], mode


def _f2_worker(rank, world):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    from piper_b200.ops import moe as M, native
    from piper_b200.parallel.fused import ShardedWeight
    from piper_b200.runtime.layout import init_distributed

    init_distributed("cuda")
    dev = torch.device("cuda", rank)
    ranks = list(range(world))
    out = {}
    # ---- F2: all-gather fused into the GEMM
    g = torch.Generator(device="cpu").manual_seed(11)
    N, K, T = 1000, 512, 384                  # N is not a multiple of the shard or tile size on purpose
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(dev)
    sw = ShardedWeight(w, ranks, None, keep_full=True)
    y = sw.linear(x)
    torch.cuda.synchronize()
    native.check_status()
    ref = x.float() @ w.float().t()
    out["f2_rel"] = ((y.float() - ref).norm() / ref.norm()).item()
    out["f2_full_equal"] = bool(torch.equal(sw.full, w))
    # second launch on the same object (scratch counters are reused), then the direct mode without a full buffer
    sw.full.zero_()
    y2 = sw.linear(x)
    torch.cuda.synchronize()
    native.check_status()
    out["f2_repeat_equal"] = bool(torch.equal(y2, y)) and bool(torch.equal(sw.full, w))
    dist.barrier()
    del sw
    N2, K2, T2 = 2304, 1024, 640               # several weight blocks and row tiles per rank
    w2 = (torch.randn(N2, K2, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    x2 = torch.randn(T2, K2, generator=g).to(torch.bfloat16).to(dev)
    ref2 = x2.float() @ w2.float().t()
    for keep in (True, False):
        sw2 = ShardedWeight(w2, ranks, None, keep_full=keep)
        yk = sw2.linear(x2)
        torch.cuda.synchronize()
        native.check_status()
        out[f"f2_rel_big_{keep}"] = ((yk.float() - ref2).norm() / ref2.norm()).item()
        if keep:
            out["f2_full_equal"] = out["f2_full_equal"] and bool(torch.equal(sw2.full, w2))
        dist.barrier()
        del sw2
    return out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_f2_ag_gemm_on_two_gpus(tmp_path):
    from tests.dist_utils import run_ranks

    res = run_ranks(2, _f2_worker, (), tmp_path, timeout=600)
    for r in res:
        assert r["f2_rel"] < 1e-2 and r["f2_full_equal"] and r["f2_repeat_equal"], r
        assert r["f2_rel_big_True"] < 1e-2 and r["f2_rel_big_False"] < 1e-2, r


@pytest.mark.parametrize("me", [0, 1, 2])
def test_f2_gathered_mode_with_local_shards_on_one_gpu(me):
    """The gather path of the all-gather GEMM, with every shard in this GPU's own memory (three "ranks")."""
    from piper_b200.ops import native

    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(5)
    N, K, T, shards = 1664, 640, 300, 3       # shards of 576 rows: 256-row weight blocks straddle shard boundaries
    rows = ((N + shards - 1) // shards + 63) // 64 * 64
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(dev)
    parts = []
    for p in range(shards):
        s_ = torch.zeros(rows, K, dtype=torch.bfloat16, device=dev)
        lo, hi = p * rows, min((p + 1) * rows, N)
        if hi > lo:
            s_[:hi - lo].copy_(w[lo:hi])
        parts.append(s_)
    full = torch.zeros(N, K, dtype=torch.bfloat16, device=dev)
    scratch = torch.zeros((N + 255) // 256 + 2, dtype=torch.int32, device=dev)
    y = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
    native.lib().ag_gemm(x, [p.data_ptr() for p in parts], me, full, scratch, y, N, rows, native.status_tensor(dev))
    torch.cuda.synchronize()
    native.check_status()
    ref = x.float() @ w.float().t()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 1e-2
    assert torch.equal(full, w)


# ------------------------------------------------------------------------------------------------------------
# Expert-parallel exchanges lowered to peer-memory kernels (dispatch gather-push, grouped GEMMs on the receive
# region, segment return, and the two backward mirrors) against the all-to-all lowering of the same DAG.
def _moe_run(rank, world, fused, steps, schedule="plain"):
    """Trains a small Qwen3-style model with a sharded expert region; returns losses, parameters, expert grads."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["PIPER_PEER_TIMEOUT_S"] = "5"
    os.environ["PIPER_FUSED"] = "1" if fused else "0"
    os.environ["PIPER_FUSED_EP"] = "force" if fused else "0"
    import torch
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.compiler.builders import build_zerobubble_schedule
    from piper_b200.models.qwen3 import PiperQwen3Model, Qwen3Config
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.ops import native

    torch.cuda.set_device(rank)
    cfg = Qwen3Config(dim=256, n_layers=3, n_heads=4, n_kv_heads=2, head_dim=64, vocab_size=1024, num_experts=8,
                      top_k=2, moe_hidden=128, max_seq_len=128)
    seq, mbs = 128, 3
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab_size, (mbs * 2 * world, seq + 1), generator=g)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    per = x.shape[0] // world
    xs, ys = x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per]
    devs = list(range(world))
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": devs}]
    if world > 1:
        sched.append({"op": "replicate", "filter": {"PP": 0}, "devices": devs, "reduce_stream": "dp_stream"})
    sched.append({"op": "shard", "filter": {"PP": 0, "EP": "*"}, "devices": devs, "stream": "ep_stream"})
    sched.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": mbs})
    if schedule == "zerobubble":
        sched += build_zerobubble_schedule(1, mbs)      # BWD_I / BWD_W split: deferred expert weight gradients
    actor = piper_setup(PiperQwen3Model, (cfg, 1, seq), optim_fn=torch.optim.Adam, optim_kwargs={"lr": 1e-3},
                        example_inputs=[xs], example_outputs=ys, model_dtype=torch.bfloat16,
                        const_attrs=PiperQwen3Model.const_attrs(cfg, seq), schedule_directives=sched, device="cuda")
    assert (actor.ep_fused is not None) == fused
    actor.debug_keep_grads = True
    losses, grads = [], None
    for it in range(steps):
        losses.append([float(v) for v in piper_exec_dag(cross_entropy_loss)])
        if it == 0:
            grads = {k: (v[1] if isinstance(v, tuple) else v).float().cpu() for k, v in actor.last_grads.items()
                     if "experts" in k}
    torch.cuda.synchronize()
    native.check_status()
    params = {k: v.float().cpu() for k, v in actor.named_parameters().items()}
    slots = actor.ep_fused.slots if fused else 0
    return {"losses": losses, "params": params, "grads": grads, "slots": slots}


def _moe_both(rank, world, steps):
    return _moe_run(rank, world, True, steps), _moe_run(rank, world, False, steps)


def _check_moe_pair(fused, base):
    assert fused["slots"] >= 1
    for a, b in zip(fused["losses"], base["losses"]):
        for u, v in zip(a, b):
            assert abs(u - v) < 3e-2, (fused["losses"], base["losses"])
    assert fused["losses"][-1][0] < fused["losses"][0][0]
    assert fused["grads"], "no expert gradients were recorded"
    for k, gf in fused["grads"].items():
        gb = base["grads"][k]
        assert gf.shape == gb.shape
        rel = ((gf - gb).norm() / (gb.norm() + 1e-12)).item()
        assert rel < 2e-2, (k, rel)
        assert (gf - gb).abs().max().item() <= 2e-2 * gb.abs().max().item() + 1e-6, k
    for k, pf in fused["params"].items():
        d = (pf - base["params"][k]).abs()
        assert d.max() <= 1.6e-2 and d.mean() < 4e-4, (k, float(d.max()), float(d.mean()))


@pytest.mark.parametrize("schedule", ["plain", "zerobubble"])
def test_fused_expert_exchange_matches_the_local_lowering_on_one_gpu(schedule):
    """Group of one rank: every kernel of the exchange runs (peers are this GPU), flags and slots are reused
    over several steps, and the result must match the lowering without an exchange."""
    fused = _moe_run(0, 1, True, 4, schedule)
    base = _moe_run(0, 1, False, 4, schedule)
    _check_moe_pair(fused, base)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_expert_exchange_matches_all_to_all_on_two_gpus(tmp_path):
    from tests.dist_utils import run_ranks

    res = run_ranks(2, _moe_both, (4,), tmp_path, timeout=900)
    for r in range(2):
        _check_moe_pair(res[r][0], res[r][1])


def test_expert_dispatch_rejects_a_region_overflow():
    """A capacity factor below the routed load: the rows for the overflowing owner are not sent and the status
    word reports a rejected argument; nothing is written out of bounds and the context stays usable."""
    from piper_b200.ops import moe as M, native
    from piper_b200.parallel.ep_fused import _Pool

    dev = torch.device("cuda")
    T, D, E, k = 1024, 128, 4, 2
    pool = _Pool([0], None, 0, 1, T, D, E, k, 0.25, dev)       # a quarter of the balanced share
    assert pool.cap_src < T * k
    x = torch.randn(T, D, device=dev).to(torch.bfloat16)
    idx = torch.zeros(T, k, dtype=torch.int32, device=dev)
    idx[:, 1] = 1
    counts = torch.tensor([T, T, 0, 0], dtype=torch.int32, device=dev)
    g_start = torch.empty_like(counts)
    g_len = torch.empty_like(counts)
    native.lib().moe_group_table(counts, E, None, g_start, g_len, torch.empty(1, dtype=torch.int32, device=dev))
    scratch = torch.zeros(2 * E + 2, dtype=torch.int32, device=dev)
    pos = torch.empty(T * k, dtype=torch.int32, device=dev)
    status = native.status_tensor(dev)
    status.zero_()
    before = pool.recv[0].clone()
    native.lib().ep_dispatch_push(x, idx, counts, g_start, scratch[:E], scratch[2 * E:], scratch[E:2 * E], pos,
                                  pool.recv_ptrs[0], pool.meta_ptrs[0], pool.flags_ptrs, pool.flags_local,
                                  pool.off(0, 1), 0, pool.off(0, 0), 1, pool.counters[0:1], 0, 1, pool.cap_src, 1.0,
                                  status, 8)
    torch.cuda.synchronize()
    with pytest.raises(native.PiperKernelError):
        native.check_status()
    assert torch.equal(pool.recv[0], before)
