"""Expert module under the name the reference's Qwen3 example imports (``BmmExperts``).

The reference pads every expert to ``tokens x top_k`` rows and runs three ``torch.bmm`` calls behind the custom
op ``piper_artifact::bmm_experts`` (``examples/models/qwen3_bmm_experts_patch.py:11-50,56-110``).  Here the same
interface is served by the ragged grouped tcgen05 GEMMs of ``piper_b200.models.qwen3.GroupedExperts``: rows arrive
sorted by expert in segments padded to 128 rows, ``num_tokens_per_expert`` gives the valid rows per segment, and
nothing is padded to capacity.  ``bmm_experts`` is the functional form on separate ``w1``/``w2``/``w3`` weights.
"""
from __future__ import annotations

import torch

from piper_b200 import ops
from piper_b200.models.qwen3 import GroupedExperts
from piper_b200.ops import moe as moe_ops


def bmm_experts(w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor, x: torch.Tensor,
                num_tokens_per_expert: torch.Tensor) -> torch.Tensor:
    """``w2[e] @ (silu(w1[e] @ x_e) * (w3[e] @ x_e))`` for every expert segment ``x_e`` of ``x``.

    ``w1``/``w3``: ``[E, F, D]``, ``w2``: ``[E, D, F]``; ``x`` holds the expert-sorted rows in 128-row-padded
    segments (the layout ``piper::moe_dispatch`` produces).
    """
    w13 = torch.cat([w1, w3], dim=1)
    g_start, g_len = moe_ops.moe_group_table(num_tokens_per_expert, w13)
    h = moe_ops.grouped_linear(x, w13, g_start, g_len)
    return moe_ops.grouped_linear(ops.swiglu(h), w2, g_start, g_len)


class BmmExperts(GroupedExperts):
    """``BmmExperts(dim, hidden_dim, num_experts)``; ``forward(x, num_tokens_per_expert)``."""

    def __init__(self, dim: int, hidden_dim: int, num_experts: int) -> None:
        super().__init__(dim, hidden_dim, num_experts)

    def forward(self, x: torch.Tensor, num_tokens_per_expert: torch.Tensor) -> torch.Tensor:
        return super().forward(x, num_tokens_per_expert)
