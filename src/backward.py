"""``src.backward`` of the reference (autograd-graph surgery for split backward, ``src/backward.py:25-169``).

Not needed here: every linear op records its weight-gradient GEMM as a deferred thunk while the input-gradient
pass runs (``piper_b200.ops.core.wgrad_store``), and the BWD_W node drains that queue.
"""
from piper_b200.ops.core import WgradStore, wgrad_store  # noqa: F401
