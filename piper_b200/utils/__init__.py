"""Utilities: kernel micro-benchmarks, clock sampling, logging helpers."""
