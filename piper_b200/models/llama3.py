"""Llama-3-style dense decoder with pipeline-stage annotations.

Same architecture family and configurations as the reference example
(``examples/models/llama3.py``: RMSNorm, RoPE, GQA attention, SwiGLU;
``debug/1b/3b/8b/70b``), written on the framework's own ops: fused QKV and
gate/up projections, rotary embedding applied for real (the reference
replaces the table by ones, ``llama3.py:137-139``), flash attention instead
of a materialised ``[B,H,S,S]`` score tensor, and the residual add fused into
the following RMSNorm.  ``forward`` wraps ``num_stages`` equal slices of the
layer stack in ``annotate("PP")`` scopes; the embedding belongs to the first
stage and the final norm and LM head to the last.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..api import annotate
from ..nn import Attention, Embedding, FeedForward, Linear, RMSNorm


@dataclass
class LlamaConfig:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    vocab_size: int = 128256
    ffn_hidden: int = 14336
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_seq_len: int = 4096

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads


LLAMA_CONFIGS = {
    # config 1 of the acceptance list: 4 layers, hidden 256, 4 heads, FFN 688, vocab 1024
    "tiny": LlamaConfig(dim=256, n_layers=4, n_heads=4, n_kv_heads=4, vocab_size=1024, ffn_hidden=688,
                        norm_eps=1e-6, rope_theta=10000.0, max_seq_len=128),
    "debug": LlamaConfig(dim=256, n_layers=8, n_heads=16, n_kv_heads=16, vocab_size=2048, ffn_hidden=768,
                         max_seq_len=2048),
    "1b": LlamaConfig(dim=2048, n_layers=16, n_heads=32, n_kv_heads=8, ffn_hidden=8192),
    "3b": LlamaConfig(dim=3072, n_layers=28, n_heads=24, n_kv_heads=8, ffn_hidden=8192),
    "8b": LlamaConfig(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_hidden=14336),
    "70b": LlamaConfig(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, ffn_hidden=28672),
}


class TransformerBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig) -> None:
        super().__init__()
        self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.attention = Attention(cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, qk_norm=False,
                                   rope_interleaved=True, norm_eps=cfg.norm_eps)
        self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.feed_forward = FeedForward(cfg.dim, cfg.ffn_hidden)

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], cos, sin, batch: int, seq: int):
        """``h`` is the residual stream and ``delta`` a branch output not yet added to it.

        Returns the new ``(h, delta)``; the pending add is folded into the next RMSNorm.
        """
        if delta is None:
            y = self.attention_norm(h)
        else:
            y, h = self.attention_norm(delta, h)
        a = self.attention(y, cos, sin, batch, seq)
        y, h = self.ffn_norm(a, h)
        return h, self.feed_forward(y)


def balanced_stage_layers(n_layers: int, num_stages: int, head_units: float = 2.3) -> list:
    """Layers per stage when the last stage's LM head + loss cost about ``head_units`` transformer layers."""
    left, out = n_layers + head_units, []
    layers_left = n_layers
    for s in range(num_stages - 1):
        take = max(1, min(layers_left - (num_stages - 1 - s), round(left / (num_stages - s))))
        out.append(take)
        left -= take
        layers_left -= take
    out.append(layers_left)
    return out


class Transformer(nn.Module):
    def __init__(self, cfg: LlamaConfig, seq_len: Optional[int] = None, num_stages: Optional[int] = None,
                 stage_layers: Optional[list] = None) -> None:
        """``stage_layers`` (layers per pipeline stage) overrides the equal split, e.g. to give the last stage,
        which also runs the LM head and the loss, fewer layers."""
        super().__init__()
        self.cfg = cfg
        self.stage_layers = list(stage_layers) if stage_layers else None
        self.seq_len = seq_len or cfg.max_seq_len
        if num_stages is None:
            from ..state import piper_metadata
            num_stages = int((piper_metadata.schedule_info or {}).get("num_stages", 1))
        self.num_stages = num_stages
        self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim)
        self.layers = nn.ModuleList(TransformerBlock(cfg) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.output = Linear(cfg.dim, cfg.vocab_size)
        self.register_buffer("rope_cos", torch.empty(self.seq_len, cfg.head_dim // 2), persistent=False)
        self.register_buffer("rope_sin", torch.empty(self.seq_len, cfg.head_dim // 2), persistent=False)

    @staticmethod
    def const_attrs(cfg: LlamaConfig, seq_len: int, device=None) -> dict:
        """The non-trainable tensors the runtime must provide by name: fp32 rotary tables."""
        cos, sin = ops.rope_tables(cfg.head_dim, seq_len, cfg.rope_theta, device=device)
        return {"rope_cos": cos, "rope_sin": sin}

    def load_const_attrs(self, seq_len: Optional[int] = None) -> None:
        c = self.const_attrs(self.cfg, seq_len or self.seq_len, self.rope_cos.device)
        self.rope_cos, self.rope_sin = c["rope_cos"].float(), c["rope_sin"].float()

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        batch, seq = tokens.shape
        n = len(self.layers)
        h = delta = None
        out = None
        bounds = [0]
        for stage in range(self.num_stages):
            bounds.append(bounds[-1] + self.stage_layers[stage] if self.stage_layers
                          else (stage + 1) * n // self.num_stages)
        for stage in range(self.num_stages):
            lo, hi = bounds[stage], bounds[stage + 1]
            with annotate("PP"):
                if stage == 0:
                    h = self.tok_embeddings(tokens.reshape(-1))
                for i in range(lo, hi):
                    h, delta = self.layers[i](h, delta, self.rope_cos, self.rope_sin, batch, seq)
                if stage == self.num_stages - 1:
                    y, h = self.norm(delta, h)
                    out = self.output(y).view(batch, seq, -1)
                elif delta is not None:
                    # one tensor crosses the stage boundary, not two
                    h = ops.residual_add(h, delta)
                    delta = None
        return out
