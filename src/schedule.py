"""``src.schedule`` of the reference, provided by ``piper_b200.compiler.schedule``."""
from piper_b200.compiler.schedule import derive_schedule_info, load_schedule_directives, load_schedule_info  # noqa: F401
