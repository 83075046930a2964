"""Two GPUs over NCCL against one GPU: the same model, data and number of steps through pipeline parallelism
(PP2, 1F1B) and through ZeRO-3 data parallelism in its NCCL lowering must reproduce the single-GPU losses and
parameters up to bf16 rounding and reduction order."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

STEPS, GLOBAL_BATCH, SEQ, MICROBATCHES = 3, 8, 128, 4


def _run(rank, world, layout):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["PIPER_FUSED"] = "0"                     # NCCL collectives, not the peer-memory kernels
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.compiler.builders import build_1f1b_schedule
    from piper_b200.models.llama3 import LlamaConfig, Transformer
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.ops import native

    torch.cuda.set_device(rank)
    cfg = LlamaConfig(dim=256, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=1024, ffn_hidden=512, max_seq_len=SEQ)
    tok = torch.randint(0, cfg.vocab_size, (GLOBAL_BATCH, SEQ + 1), generator=torch.Generator().manual_seed(11))
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    stages, mbs = 1, MICROBATCHES
    if layout == "single":
        sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0]}]
    elif layout == "pp2":
        stages = 2
        sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0]}, {"op": "place", "filter": {"PP": 1}, "devices": [1]}]
    else:                                               # zero3 over two replicas: half the batch, half the microbatches
        per = GLOBAL_BATCH // world
        x, y, mbs = x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per], MICROBATCHES // world
        sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0, 1]},
                 {"op": "replicate", "filter": {"PP": 0}, "devices": [0, 1], "reduce_stream": "dp_stream",
                  "gather_stream": "gather_stream", "shard_params": True, "bucket_size": 1}]
    sched.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": mbs})
    if layout == "pp2":
        sched += build_1f1b_schedule(2, mbs)
    actor = piper_setup(Transformer, (cfg, SEQ, stages), optim_fn=torch.optim.Adam, optim_kwargs={"lr": 1e-3},
                        example_inputs=[x], example_outputs=y, model_dtype=torch.bfloat16,
                        const_attrs=Transformer.const_attrs(cfg, SEQ), schedule_directives=sched, device="cuda")
    assert actor.fused is None
    losses = []
    for _ in range(STEPS):
        out = piper_exec_dag(cross_entropy_loss)
        losses.append(sorted(float(v) for v in out) if out else [])
    torch.cuda.synchronize()
    native.check_status()
    return {"losses": losses, "params": {k: v.float().cpu() for k, v in actor.named_parameters().items()}}


def _both(rank, world):
    return {"pp2": _run(rank, world, "pp2"), "zero3": _run(rank, world, "zero3")}


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pp2_and_zero3_over_nccl_match_one_gpu(tmp_path):
    from tests.dist_utils import run_ranks

    (tmp_path / "one").mkdir()
    (tmp_path / "two").mkdir()
    single = run_ranks(1, _run, ("single",), tmp_path / "one", timeout=600)[0]
    two = run_ranks(2, _both, (), tmp_path / "two", timeout=900)
    want = [sum(l) / len(l) for l in single["losses"]]
    assert want[-1] < want[0]

    # pipeline: the last stage's rank holds the losses; the union of both ranks' parameters is the model
    pp = [r["pp2"] for r in two]
    got = [sum(l) / len(l) for l in next(r["losses"] for r in pp if r["losses"][0])]
    params = {**pp[0]["params"], **pp[1]["params"]}
    assert set(params) == set(single["params"])
    # data parallel: each replica saw half of the microbatches; parameters are identical on both replicas
    z = [r["zero3"] for r in two]
    zl = [(sum(a) + sum(b)) / (len(a) + len(b)) for a, b in zip(z[0]["losses"], z[1]["losses"])]
    for k in z[0]["params"]:
        assert torch.equal(z[0]["params"][k], z[1]["params"][k]), k
    for name, losses, p in (("pp2", got, params), ("zero3", zl, z[0]["params"])):
        for a, b in zip(losses, want):
            assert abs(a - b) < 2e-2, (name, losses, want)
        for k, ref in single["params"].items():
            d = (p[k] - ref).abs()
            assert d.max() <= 8e-3 and d.mean() < 2e-4, (name, k, float(d.max()), float(d.mean()))
