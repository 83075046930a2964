"""Bundled model families: Llama-3-style dense decoders and Qwen3-style MoE decoders."""
