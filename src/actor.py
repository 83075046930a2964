"""``src.actor`` of the reference: the per-GPU executor host lives in ``piper_b200.runtime.actor``.

There are no Ray actors here; ``PiperActor`` is an ordinary object owned by the one process that drives its GPU.
"""
from piper_b200.runtime.actor import PiperActor, StageBucket  # noqa: F401
