"""Qwen3-style mixture-of-experts decoder with pipeline-stage and expert-parallel annotations.

Architecture family of the reference example (``examples/models/qwen3.py``: GQA attention with
QK-RMSNorm and rotary embedding, top-k softmax router with renormalised weights, SwiGLU experts, no shared
expert; configurations 9M ... 72B including ``30B-A3B``), built on this framework's ops instead of
torchtitan modules.  ``forward`` wraps equal layer slices in ``annotate("PP")``; inside each MoE layer only
the expert computation is wrapped in ``annotate("EP")``, so a ``shard`` directive on ``{"PP": i, "EP": "*"}``
turns its boundaries into token exchanges and partitions the expert weights over the group.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..api import annotate
from ..nn import Attention, Embedding, FeedForward, Linear, RMSNorm
from ..ops import moe as moe_ops

PP_TAG = "PP"
EP_TAG = "EP"


@dataclass
class Qwen3Config:
    dim: int = 2048
    n_layers: int = 48
    n_heads: int = 32
    n_kv_heads: int = 4
    head_dim: int = 128
    vocab_size: int = 151936
    num_experts: int = 128
    top_k: int = 8
    moe_hidden: int = 768
    ffn_hidden: int = 6144          # dense layers (moe disabled)
    moe_enabled: bool = True
    norm_topk_prob: bool = True
    norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    max_seq_len: int = 4096
    # Noisy top-k gating with frozen noise: a fixed N(0, std) table [seq, experts] added to the router logits.
    # A randomly initialised deep MoE sends almost every token to the same few experts (the residual streams of
    # different positions are strongly correlated before any training); benchmark runs set a std that dominates
    # the initial logits so that the load over experts is near-uniform from the first step.  0 disables it.
    router_jitter_std: float = 0.0


QWEN3_CONFIGS = {
    "9M": Qwen3Config(dim=256, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=64, vocab_size=2048, num_experts=8,
                      top_k=2, moe_hidden=256, max_seq_len=1024),
    "1B": Qwen3Config(dim=1024, n_layers=16, n_heads=16, n_kv_heads=4, head_dim=128, num_experts=32, top_k=4,
                      moe_hidden=512),
    "9B": Qwen3Config(dim=2048, n_layers=24, n_heads=32, n_kv_heads=4, head_dim=128, num_experts=64, top_k=8,
                      moe_hidden=768),
    "30B-A3B": Qwen3Config(),
    "30-A3B-half": Qwen3Config(n_layers=24),
    "48B": Qwen3Config(dim=2560, n_layers=48, n_heads=32, n_kv_heads=4, num_experts=128, top_k=8, moe_hidden=1024),
    "72B": Qwen3Config(dim=3072, n_layers=56, n_heads=48, n_kv_heads=8, num_experts=128, top_k=8, moe_hidden=1280),
}


def create_qwen3_config(name: str) -> Qwen3Config:
    return QWEN3_CONFIGS[name]


class GroupedExperts(nn.Module):
    """SwiGLU experts with stacked weights: w13 [E, 2F, D] (gate rows then up rows) and w2 [E, D, F]."""

    def __init__(self, dim: int, hidden: int, num_experts: int) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.w13 = nn.Parameter(torch.empty(num_experts, 2 * hidden, dim))
        self.w2 = nn.Parameter(torch.empty(num_experts, dim, hidden))

    def forward(self, rows: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        """``counts`` holds one entry per (source, local expert) group; the weights' leading dim is the local expert count."""
        g_start, g_len = moe_ops.moe_group_table(counts, self.w13)
        h = moe_ops.grouped_linear(rows, self.w13, g_start, g_len)
        return moe_ops.grouped_linear(ops.swiglu(h), self.w2, g_start, g_len)


class MoE(nn.Module):
    def __init__(self, cfg: Qwen3Config) -> None:
        super().__init__()
        self.top_k, self.renorm = cfg.top_k, cfg.norm_topk_prob
        self.gate = Linear(cfg.dim, cfg.num_experts)
        self.experts = GroupedExperts(cfg.dim, cfg.moe_hidden, cfg.num_experts)

    def forward(self, x: torch.Tensor, jitter: Optional[torch.Tensor] = None) -> torch.Tensor:
        logits = self.gate(x)
        if jitter is not None:
            logits = logits + jitter
        weights, idx, counts = moe_ops.moe_route(logits, self.top_k, self.renorm)
        rows, pos, g_start, g_len, ep_counts = moe_ops.moe_dispatch(x, idx, counts)
        with annotate(EP_TAG):
            out_rows = self.experts(rows, ep_counts)
        return moe_ops.moe_combine(out_rows, pos, weights, g_start, g_len, counts)


class Qwen3Block(nn.Module):
    def __init__(self, cfg: Qwen3Config) -> None:
        super().__init__()
        self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.attention = Attention(cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, qk_norm=True,
                                   rope_interleaved=False, norm_eps=cfg.norm_eps)
        self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.moe = MoE(cfg) if cfg.moe_enabled else None
        self.feed_forward = None if cfg.moe_enabled else FeedForward(cfg.dim, cfg.ffn_hidden)

    def forward(self, h, delta, cos, sin, batch: int, seq: int, jitter=None):
        if delta is None:
            y = self.attention_norm(h)
        else:
            y, h = self.attention_norm(delta, h)
        a = self.attention(y, cos, sin, batch, seq)
        y, h = self.ffn_norm(a, h)
        return h, (self.moe(y, jitter) if self.moe is not None else self.feed_forward(y))


class PiperQwen3Model(nn.Module):
    def __init__(self, cfg: Qwen3Config, num_stages: Optional[int] = None, seq_len: Optional[int] = None) -> None:
        super().__init__()
        self.cfg = cfg
        self.seq_len = seq_len or cfg.max_seq_len
        if num_stages is None:
            from ..state import piper_metadata
            info = piper_metadata.schedule_info or {}
            num_stages = int(info.get("num_stages", info.get("pp_degree", 2)))
        self.num_stages = num_stages
        self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim)
        self.layers = nn.ModuleList(Qwen3Block(cfg) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.output = Linear(cfg.dim, cfg.vocab_size)
        self.register_buffer("rope_cos", torch.empty(self.seq_len, cfg.head_dim // 2), persistent=False)
        self.register_buffer("rope_sin", torch.empty(self.seq_len, cfg.head_dim // 2), persistent=False)
        self.use_jitter = cfg.router_jitter_std > 0 and cfg.moe_enabled
        if self.use_jitter:
            self.register_buffer("router_jitter", torch.empty(self.seq_len, cfg.num_experts), persistent=False)

    @staticmethod
    def const_attrs(cfg: Qwen3Config, seq_len: int, device=None) -> dict:
        cos, sin = ops.rope_tables(cfg.head_dim, seq_len, cfg.rope_theta, device=device)
        out = {"rope_cos": cos, "rope_sin": sin}
        if cfg.router_jitter_std > 0 and cfg.moe_enabled:
            g = torch.Generator().manual_seed(20240229)
            noise = torch.randn(seq_len, cfg.num_experts, generator=g) * cfg.router_jitter_std
            out["router_jitter"] = noise.to(torch.bfloat16).to(device) if device is not None else noise.to(torch.bfloat16)
        return out

    def load_const_attrs(self, seq_len: Optional[int] = None) -> None:
        c = self.const_attrs(self.cfg, seq_len or self.seq_len, self.rope_cos.device)
        self.rope_cos, self.rope_sin = c["rope_cos"].float(), c["rope_sin"].float()
        if self.use_jitter:
            self.router_jitter = c["router_jitter"].to(self.rope_cos.device)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        batch, seq = tokens.shape
        n = len(self.layers)
        h = delta = out = None
        jitter = None
        if self.use_jitter:
            jitter = self.router_jitter if batch == 1 else self.router_jitter.repeat(batch, 1)
        for stage in range(self.num_stages):
            lo, hi = stage * n // self.num_stages, (stage + 1) * n // self.num_stages
            with annotate(PP_TAG):
                if stage == 0:
                    h = self.tok_embeddings(tokens.reshape(-1))
                for i in range(lo, hi):
                    h, delta = self.layers[i](h, delta, self.rope_cos, self.rope_sin, batch, seq, jitter)
                if stage == self.num_stages - 1:
                    y, h = self.norm(delta, h)
                    out = self.output(y).view(batch, seq, -1)
                elif delta is not None:
                    h = ops.residual_add(h, delta)
                    delta = None
        return out
