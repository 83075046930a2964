"""piper_b200: a Blackwell-native programmable distributed-training framework.

Public surface (the same names the reference exposes from ``src.piper`` /
``src.compile``): ``annotate``, ``piper_setup``, ``piper_exec_dag``, the
``piper`` Dynamo backend (registered on import), schedule loading and the
schedule builders.
"""
from .api import annotate, compile_training_dags, piper  # noqa: F401  (registers the Dynamo backend)
from .state import piper_metadata  # noqa: F401

__all__ = ["annotate", "piper_setup", "piper_exec_dag", "piper_metadata", "compile_training_dags"]


def piper_setup(*args, **kwargs):
    from .engine import piper_setup as _impl
    return _impl(*args, **kwargs)


def piper_exec_dag(*args, **kwargs):
    from .engine import piper_exec_dag as _impl
    return _impl(*args, **kwargs)
