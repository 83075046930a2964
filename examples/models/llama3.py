"""Llama-3 example model: see ``piper_b200.models.llama3``."""
from piper_b200.models.llama3 import LLAMA_CONFIGS, LlamaConfig, Transformer, TransformerBlock  # noqa: F401
