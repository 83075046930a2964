"""``src.state`` of the reference, provided by ``piper_b200.state``."""
from piper_b200.state import LOG_LEVEL, PiperMetadata, create_logger, piper_metadata  # noqa: F401
