"""Model building blocks on top of ``torch.ops.piper.*``."""
from .layers import (Attention, CrossEntropyLoss, Embedding, FeedForward, Linear, RMSNorm, cross_entropy_loss)

__all__ = ["Linear", "RMSNorm", "Embedding", "Attention", "FeedForward", "CrossEntropyLoss", "cross_entropy_loss"]
