"""Fused compute+collective kernels: bounded peer wait (1 GPU) and equivalence with the NCCL lowering (2 GPUs)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_f1_peer_wait_times_out_cleanly():
    """A peer flag that nothing sets: the kernel gives up after the deadline, reports status 2, context stays usable."""
    from piper_b200.ops import native

    lib = native.lib()
    dev = torch.device("cuda")
    n = 4096
    grads = [torch.ones(n, device=dev), torch.ones(n, device=dev)]
    params = [torch.zeros(n, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    flags = [torch.zeros(4, device=dev, dtype=torch.int64) for _ in range(2)]
    ptr = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    master = torch.zeros(n // 2, device=dev)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    status = native.status_tensor()
    status.zero_()
    lib.f1_rs_adam_ag(ptr(grads), ptr(params), ptr(flags), master, m, v, 0, 2, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1,
                      1.0, counter, status, 0.2, 8)
    torch.cuda.synchronize()
    with pytest.raises(native.PiperCommTimeout):
        native.check_status()
    assert int(status.item()) == 0          # reset by check_status
    assert torch.equal(master, torch.zeros_like(master))   # nothing was updated
    x = torch.ones(8, device=dev) * 2       # the context still works
    assert float(x.sum()) == 16.0


def _dp_worker(rank, world, fused, steps):
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
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": devs},
             {"op": "replicate", "filter": {"PP": 0}, "devices": devs, "reduce_stream": "dp_stream"},
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
    return {"losses": losses, "params": params}


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_f1_matches_nccl_allreduce_adam_on_two_gpus(tmp_path):
    from tests.dist_utils import run_ranks

    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    fused = run_ranks(2, _dp_worker, (True, 4), tmp_path / "a", timeout=600)
    base = run_ranks(2, _dp_worker, (False, 4), tmp_path / "b", timeout=600)
    # replicas agree with each other bit-for-bit after the fused all-gather
    for k in fused[0]["params"]:
        assert torch.equal(fused[0]["params"][k], fused[1]["params"][k]), k
    # and with the NCCL lowering up to reduction order and bf16 rounding
    for k, p in fused[0]["params"].items():
        d = (p - base[0]["params"][k]).abs()
        assert d.max() <= 8e-3 and d.mean() < 2e-4, (k, float(d.max()), float(d.mean()))
    assert abs(fused[0]["losses"][-1][0] - base[0]["losses"][-1][0]) < 5e-2
    assert fused[0]["losses"][-1][0] < fused[0]["losses"][0][0]


def _f2_f3_worker(rank, world):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    from piper_b200.ops import moe as M, native
    from piper_b200.parallel.fused import FusedExpertExchange, ShardedWeight
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
    # ---- F3: dispatch push -> (identity expert x2) -> combine pull
    Tt, D, E, k = 512, 256, 8, 2
    g2 = torch.Generator(device="cpu").manual_seed(100 + rank)
    xt = torch.randn(Tt, D, generator=g2).to(torch.bfloat16).to(dev)
    logits = torch.randn(Tt, E, generator=g2).to(torch.bfloat16).to(dev)
    weights, idx, counts = M.moe_route(logits, k, True)
    ex = FusedExpertExchange(ranks, None, Tt, D, E, k, timeout_s=20.0)
    for it in range(2):                        # two epochs: flags and buffers are reused
        rows, pos, g_start, g_len, recv_counts = ex.dispatch(xt, idx, counts)
        torch.cuda.synchronize()
        native.check_status()
        # received counts must equal what every source routed to this rank's experts
        all_counts = [torch.empty_like(counts) for _ in ranks]
        dist.all_gather(all_counts, counts)
        El = E // world
        want = torch.stack([c[rank * El:(rank + 1) * El] for c in all_counts]).reshape(-1)
        out[f"f3_counts_ok_{it}"] = bool(torch.equal(recv_counts, want))
        # "expert": double every valid row
        ex.out_rows.copy_(rows * 2)
        got = ex.combine(pos, weights, Tt)
        torch.cuda.synchronize()
        native.check_status()
        refc = 2 * xt.float()
        out[f"f3_rel_{it}"] = ((got.float() - refc).norm() / refc.norm()).item()
        dist.barrier()
    return out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_f2_ag_gemm_and_f3_dispatch_combine_on_two_gpus(tmp_path):
    from tests.dist_utils import run_ranks

    res = run_ranks(2, _f2_f3_worker, (), tmp_path, timeout=600)
    for r in res:
        assert r["f2_rel"] < 1e-2 and r["f2_full_equal"] and r["f2_repeat_equal"], r
        assert r["f2_rel_big_True"] < 1e-2 and r["f2_rel_big_False"] < 1e-2, r
        for it in range(2):
            assert r[f"f3_counts_ok_{it}"], r
            assert r[f"f3_rel_{it}"] < 1.5e-2, r


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
