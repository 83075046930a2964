"""Compute ops of the framework: ``torch.ops.piper.*`` custom ops backed by sm_100a kernels."""
from . import native
from .core import (
    add_rmsnorm,
    attention,
    cross_entropy,
    embedding,
    grad_sinks,
    linear,
    qk_rope,
    residual_add,
    rmsnorm,
    rope_tables,
    swiglu,
    wgrad_store,
)

__all__ = [
    "native", "linear", "rmsnorm", "add_rmsnorm", "qk_rope", "residual_add", "rope_tables", "attention", "swiglu",
    "embedding", "cross_entropy", "grad_sinks", "wgrad_store",
]
