"""Baseline runner: DeepSpeed pipeline + ZeRO on the evaluation's MoE shapes with mock tokens.

A plain-PyTorch Qwen3-style MoE decoder (RMSNorm, GQA attention with QK-norm through SDPA, top-k softmax router,
per-expert SwiGLU MLPs) is cut into ``--pp`` pipeline stages with ``deepspeed.pipe.PipelineModule`` and trained
for ``--steps`` steps on uniform-random tokens; tokens/s over the steps after the warm-up is printed in the
``throughput tokens/s: N`` form the evaluation driver parses.  DeepSpeed is not part of this repository; without
it the script says so and exits with code 3.  Launch: ``deepspeed --num_gpus=N artifact/run_deepspeed.py …``.
Counterpart of the reference artifact's ``artifact/run_deepspeed.py:274-621``.
"""
from __future__ import annotations

import argparse
import sys
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

# name -> dict(layers, dim, heads, kv_heads, head_dim, experts, top_k, ffn, vocab, micro_bs, global_bs, seq_len)
MODEL_CONFIGS = {
    "qwen3_1b": dict(layers=16, dim=1024, heads=16, kv_heads=4, head_dim=128, experts=32, top_k=4, ffn=512,
                     vocab=151936, micro_bs=4, global_bs=32, seq_len=512),
    "qwen3_9b": dict(layers=32, dim=2048, heads=32, kv_heads=4, head_dim=128, experts=64, top_k=8, ffn=768,
                     vocab=151936, micro_bs=4, global_bs=32, seq_len=512),
    "qwen3_30b_a3b": dict(layers=48, dim=2048, heads=32, kv_heads=4, head_dim=128, experts=128, top_k=8, ffn=768,
                          vocab=151936, micro_bs=1, global_bs=16, seq_len=4096),
}


class MockTokens(torch.utils.data.Dataset):
    """Uniform-random token sequences; labels are the inputs shifted by one."""

    def __init__(self, vocab: int, seq_len: int, samples: int, seed: int) -> None:
        g = torch.Generator().manual_seed(seed)
        self.data = torch.randint(0, vocab, (samples, seq_len + 1), generator=g)

    def __len__(self) -> int:
        return self.data.shape[0]

    def __getitem__(self, i: int):
        row = self.data[i]
        return row[:-1], row[1:]


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def _rope(x, theta: float = 1e6):
    b, h, s, d = x.shape
    inv = 1.0 / theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d)
    ang = torch.arange(s, device=x.device, dtype=torch.float32)[:, None] * inv[None]
    cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)


class Block(nn.Module):
    def __init__(self, c: dict) -> None:
        super().__init__()
        self.c = c
        d, hd = c["dim"], c["head_dim"]
        self.n1, self.n2 = RMSNorm(d), RMSNorm(d)
        self.qn, self.kn = RMSNorm(hd), RMSNorm(hd)
        self.wq = nn.Linear(d, c["heads"] * hd, bias=False)
        self.wkv = nn.Linear(d, 2 * c["kv_heads"] * hd, bias=False)
        self.wo = nn.Linear(c["heads"] * hd, d, bias=False)
        self.gate = nn.Linear(d, c["experts"], bias=False)
        self.w13 = nn.Parameter(torch.randn(c["experts"], 2 * c["ffn"], d) * 0.02)
        self.w2 = nn.Parameter(torch.randn(c["experts"], d, c["ffn"]) * 0.02)

    def forward(self, x):
        c, (b, s, _) = self.c, x.shape
        h = self.n1(x)
        q = self.qn(self.wq(h).view(b, s, c["heads"], c["head_dim"])).transpose(1, 2)
        k, v = self.wkv(h).view(b, s, 2, c["kv_heads"], c["head_dim"]).unbind(2)
        k = self.kn(k).transpose(1, 2)
        att = F.scaled_dot_product_attention(_rope(q), _rope(k), v.transpose(1, 2), is_causal=True, enable_gqa=True)
        x = x + self.wo(att.transpose(1, 2).reshape(b, s, -1))
        h = self.n2(x).reshape(b * s, -1)
        w, idx = torch.topk(F.softmax(self.gate(h).float(), dim=-1), c["top_k"], dim=-1)
        out = torch.zeros_like(h)
        flat_idx, order = idx.reshape(-1).sort()
        rows = order // c["top_k"]
        counts = torch.bincount(flat_idx, minlength=c["experts"]).tolist()
        start = 0
        for e, n in enumerate(counts):                      # ragged per-expert SwiGLU
            if n:
                r = rows[start:start + n]
                a, g = (h[r] @ self.w13[e].t()).chunk(2, dim=-1)
                y = (F.silu(a) * g) @ self.w2[e].t()
                out.index_add_(0, r, y * w.reshape(-1)[order[start:start + n], None].to(y.dtype))
            start += n
        return x + out.view(b, s, -1)


class Embed(nn.Module):
    def __init__(self, c: dict) -> None:
        super().__init__()
        self.emb = nn.Embedding(c["vocab"], c["dim"])

    def forward(self, tokens):
        return self.emb(tokens)


class Head(nn.Module):
    def __init__(self, c: dict) -> None:
        super().__init__()
        self.norm, self.out = RMSNorm(c["dim"]), nn.Linear(c["dim"], c["vocab"], bias=False)

    def forward(self, x):
        return self.out(self.norm(x))


def _loss(logits, labels):
    return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), labels.reshape(-1))


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--model", choices=tuple(MODEL_CONFIGS), default="qwen3_1b")
    p.add_argument("--pp", type=int, default=4)
    p.add_argument("--dp", type=int, default=2)
    p.add_argument("--ep", type=int, default=1)
    p.add_argument("--zero-stage", type=int, default=1, choices=(0, 1, 2, 3))
    p.add_argument("--schedule", choices=("1f1b",), default="1f1b")
    p.add_argument("--micro-bs", type=int, default=None)
    p.add_argument("--global-bs", type=int, default=None)
    p.add_argument("--seq-len", type=int, default=None)
    p.add_argument("--local_rank", type=int, default=-1)
    p.add_argument("--steps", type=int, default=8)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--seed", type=int, default=42)
    a = p.parse_args(argv)
    try:
        import deepspeed
        from deepspeed.pipe import LayerSpec, PipelineModule
    except ImportError:
        print("run_deepspeed: the deepspeed package is not installed", file=sys.stderr)
        return 3

    c = dict(MODEL_CONFIGS[a.model])
    for key, val in (("micro_bs", a.micro_bs), ("global_bs", a.global_bs), ("seq_len", a.seq_len)):
        if val is not None:
            c[key] = val
    if a.pp > 1 and a.zero_stage > 1:
        raise SystemExit("DeepSpeed pipeline parallelism supports ZeRO stages 0 and 1 only")
    deepspeed.init_distributed()
    torch.manual_seed(a.seed)
    accum = c["global_bs"] // (c["micro_bs"] * a.dp)
    specs = [LayerSpec(Embed, c)] + [LayerSpec(Block, c) for _ in range(c["layers"])] + [LayerSpec(Head, c)]
    model = PipelineModule(layers=specs, num_stages=a.pp, loss_fn=_loss, partition_method="parameters")
    ds_config = {"train_batch_size": c["global_bs"], "train_micro_batch_size_per_gpu": c["micro_bs"],
                 "gradient_accumulation_steps": accum, "bf16": {"enabled": True},
                 "zero_optimization": {"stage": a.zero_stage},
                 "optimizer": {"type": "Adam", "params": {"lr": 1e-4}}, "steps_per_print": 1 << 30}
    data = MockTokens(c["vocab"], c["seq_len"], c["global_bs"] * (a.steps + a.warmup), a.seed)
    engine, _, _, _ = deepspeed.initialize(model=model, config=ds_config, training_data=data,
                                           model_parameters=[q for q in model.parameters() if q.requires_grad])
    times = []
    for step in range(a.steps + a.warmup):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        loss = engine.train_batch()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if step >= a.warmup:
            times.append(dt)
        if engine.global_rank == 0:
            print(f"[step {step}] loss={float(loss):.4f} time={dt:.3f}s", flush=True)
    if engine.global_rank == 0 and times:
        print(f"throughput tokens/s: {c['global_bs'] * c['seq_len'] / (sum(times) / len(times)):.1f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
