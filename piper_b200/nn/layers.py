"""``nn.Module`` wrappers of the custom ops.

Activations are kept two-dimensional, ``[tokens, features]`` with
``tokens = batch * seq``, from the embedding to the logits; batch and
sequence length travel as Python ints to the ops that need them.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import ops


class Linear(nn.Module):
    """y = x W^T with W stored ``[out_features, in_features]`` (no bias)."""

    def __init__(self, in_features: int, out_features: int) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        """Without ``residual``: norm(x).  With it: returns (norm(x + residual), x + residual)."""
        if residual is None:
            return ops.rmsnorm(x, self.weight, self.eps)
        return ops.add_rmsnorm(x, residual, self.weight, self.eps)


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, dim: int) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_embeddings, dim))

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return ops.embedding(tokens, self.weight)


class Attention(nn.Module):
    """Causal grouped-query self-attention with a fused QKV projection, optional QK-RMSNorm, and RoPE."""

    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, head_dim: int, qk_norm: bool = False,
                 rope_interleaved: bool = True, norm_eps: float = 1e-6) -> None:
        super().__init__()
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.rope_interleaved, self.norm_eps = rope_interleaved, norm_eps
        self.wqkv = Linear(dim, (n_heads + 2 * n_kv_heads) * head_dim)
        self.wo = Linear(n_heads * head_dim, dim)
        self.q_norm = RMSNorm(head_dim, norm_eps) if qk_norm else None
        self.k_norm = RMSNorm(head_dim, norm_eps) if qk_norm else None

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        qkv = self.wqkv(x)
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        qkv = ops.qk_rope(qkv, cos, sin, qw, kw, seq, self.n_heads, self.n_kv_heads, self.head_dim,
                          self.rope_interleaved, self.norm_eps)
        out = ops.attention(qkv, batch, seq, self.n_heads, self.n_kv_heads, self.head_dim,
                            1.0 / math.sqrt(self.head_dim))
        return self.wo(out)


class FeedForward(nn.Module):
    """SwiGLU MLP with the gate and up projections fused into one weight ``w13 = [w1; w3]``."""

    def __init__(self, dim: int, hidden: int) -> None:
        super().__init__()
        self.w13 = Linear(dim, 2 * hidden)
        self.w2 = Linear(hidden, dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w2(ops.swiglu(self.w13(x)))


def cross_entropy_loss(output: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean token cross-entropy of ``[.., V]`` logits; the fused kernel never materialises fp32 probabilities."""
    return ops.cross_entropy(output.reshape(-1, output.shape[-1]), labels.reshape(-1), ignore_index, "mean")


class CrossEntropyLoss(nn.Module):
    def __init__(self, ignore_index: int = -100) -> None:
        super().__init__()
        self.ignore_index = ignore_index

    def forward(self, output: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        return cross_entropy_loss(output, labels, self.ignore_index)
