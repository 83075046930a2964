"""``src.coordinator`` of the reference, provided by ``piper_b200.runtime.launcher``."""
from piper_b200.runtime.launcher import Coordinator, PiperProgramCoordinator  # noqa: F401
