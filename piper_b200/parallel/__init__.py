"""Parallelism building blocks: symmetric memory, fused compute+collective paths, expert-parallel exchange."""
