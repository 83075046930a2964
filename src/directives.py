"""``src.directives`` of the reference, provided by ``piper_b200.compiler.directives``."""
from piper_b200.compiler.directives import *  # noqa: F401,F403
from piper_b200.compiler.directives import (_insert_reduce_scatter_comm_nodes, _insert_shard_a2a_comm_nodes,  # noqa: F401
                                            _match_filter, _normalize_filter_spec)
