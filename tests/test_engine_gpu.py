"""The engine on a GPU: a small bf16 Llama through piper_setup / piper_exec_dag against an fp32 CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_gpu_training_step_matches_fp32_oracle_and_learns():
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.models.llama3 import LlamaConfig, Transformer
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.ops import native
    from piper_b200.runtime.storage import materialize_module

    cfg = LlamaConfig(dim=512, n_layers=4, n_heads=8, n_kv_heads=4, vocab_size=4096, ffn_hidden=1536,
                      norm_eps=1e-5, rope_theta=10000.0, max_seq_len=256)
    seq = 256
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (4, seq + 1), generator=g)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    from piper_b200.compiler.builders import build_1f1b_schedule
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0]},
             {"op": "place", "filter": {"PP": 1}, "devices": [0]},
             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2}]
    before = native.lib().kernel_launch_count()
    actor = piper_setup(Transformer, (cfg, seq, 2), optim_fn=torch.optim.Adam, optim_kwargs={"lr": 1e-3},
                        example_inputs=[x], example_outputs=y, model_dtype=torch.bfloat16,
                        const_attrs=Transformer.const_attrs(cfg, seq), schedule_directives=sched, device="cuda")
    actor.debug_keep_grads = True
    first = [float(v) for v in piper_exec_dag(cross_entropy_loss)]
    grads = {k: v.float().cpu() for k, v in actor.last_grads.items()}
    for _ in range(8):
        last = [float(v) for v in piper_exec_dag(cross_entropy_loss)]
    native.check_status()
    assert native.lib().kernel_launch_count() > before

    # the CUDA generator differs from the CPU one, so the oracle takes the GPU's initial weights
    ref = Transformer(cfg, seq, 1)
    ref.load_const_attrs()
    # re-create initial weights on the GPU with the same name-keyed rule and move them over
    from piper_b200.runtime.storage import init_tensor
    with torch.no_grad():
        for name, p in ref.named_parameters():
            p.copy_(init_tensor(name, p.shape, torch.bfloat16, torch.device("cuda")).float().cpu())
    loss = cross_entropy_loss(ref(x), y)
    loss.backward()
    assert abs(sum(first) / len(first) - float(loss.detach())) < 3e-2
    worst = 0.0
    for n_, p in ref.named_parameters():
        a, b = grads[n_], p.grad
        rel = ((a - b).norm() / (b.norm() + 1e-12)).item()
        worst = max(worst, rel)
    assert worst < 8e-2, worst
    assert sum(last) < sum(first) - 0.5, (first, last)


def test_bounded_host_run_ahead_gives_the_same_losses(monkeypatch):
    """PIPER_MAX_RUN_AHEAD makes the launch-plan executor wait for node i - n before it issues node i; the
    result of a step does not depend on it."""
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.models.llama3 import LlamaConfig, Transformer
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.ops import native

    cfg = LlamaConfig(dim=256, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=1024, ffn_hidden=512, max_seq_len=128)
    seq = 128
    tok = torch.randint(0, cfg.vocab_size, (4, seq + 1), generator=torch.Generator().manual_seed(3))
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0]}, {"op": "place", "filter": {"PP": 1}, "devices": [0]},
             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 4}]
    runs = []
    for ahead in ("0", "1"):
        monkeypatch.setenv("PIPER_MAX_RUN_AHEAD", ahead)
        actor = piper_setup(Transformer, (cfg, seq, 2), optim_fn=torch.optim.Adam, optim_kwargs={"lr": 1e-3},
                            example_inputs=[x], example_outputs=y, model_dtype=torch.bfloat16,
                            const_attrs=Transformer.const_attrs(cfg, seq), schedule_directives=sched, device="cuda")
        runs.append([[float(v) for v in piper_exec_dag(cross_entropy_loss)] for _ in range(3)])
        assert actor._plan not in (None, False)          # the C++ executor ran the steps
        native.check_status()
    for a, b in zip(runs[0], runs[1]):
        assert all(abs(u - v) < 2e-3 for u, v in zip(a, b)), (a, b)
