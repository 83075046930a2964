"""``src.zero`` of the reference, provided by ``piper_b200.compiler.zero``."""
from piper_b200.compiler.zero import add_inter_chain_temporal_edges, prune_zero_lifetimes  # noqa: F401

_prune_zero_lifetime_metadata = prune_zero_lifetimes
_add_inter_chain_temporal_edges = add_inter_chain_temporal_edges
