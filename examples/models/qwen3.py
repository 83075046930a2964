"""Qwen3 MoE example model: see ``piper_b200.models.qwen3``."""
from piper_b200.models.qwen3 import (QWEN3_CONFIGS, GroupedExperts, MoE, PiperQwen3Model, Qwen3Config,  # noqa: F401
                                     create_qwen3_config)
