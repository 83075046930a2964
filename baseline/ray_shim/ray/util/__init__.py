from . import placement_group as _pg_mod  # noqa: F401
from . import scheduling_strategies  # noqa: F401
from .placement_group import placement_group, placement_group_table, remove_placement_group  # noqa: F401


def get_node_ip_address() -> str:
    return "127.0.0.1"
