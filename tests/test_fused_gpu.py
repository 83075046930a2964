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
