"""``src.ordering`` of the reference, provided by ``piper_b200.compiler.ordering``."""
from piper_b200.compiler.ordering import (resolve_default_stream_order, resolve_total_order_per_stream,  # noqa: F401
                                          serial_topological_order)

_serial_topological_order = serial_topological_order
_resolve_default_stream_order = resolve_default_stream_order
