"""``src.compile.piper_setup`` of the reference, provided by ``piper_b200.engine``."""
from piper_b200.engine import piper_setup  # noqa: F401
