"""Stand-in ``ray`` package used only when the real one is not installed (see ``_core``)."""
from . import _core, exceptions, util  # noqa: F401
from ._core import ObjectRef, get, get_actor, kill, put, remote, wait  # noqa: F401

__version__ = "0.0-shim"
_initialized = False


def init(*args, **kwargs):
    global _initialized
    _core.start()
    _initialized = True
    return None


def is_initialized() -> bool:
    return _initialized


def shutdown() -> None:
    global _initialized
    _initialized = False
