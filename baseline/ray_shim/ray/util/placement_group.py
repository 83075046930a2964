"""Placement groups carry no information here: which process hosts an actor is decided by the job's placement
function (one process per GPU already exists when the job starts)."""
from .._core import put


class PlacementGroup:
    def __init__(self, bundles, strategy: str = "PACK", name: str = "") -> None:
        self.bundle_specs, self.strategy, self.name = list(bundles), strategy, name

    def ready(self):
        return put(self)

    def wait(self, timeout_seconds=None) -> bool:
        return True


def placement_group(bundles, strategy: str = "PACK", name: str = "", **_):
    return PlacementGroup(bundles, strategy, name)


def placement_group_table(pg=None) -> dict:
    if pg is None:
        return {}
    return {"bundles": {i: b for i, b in enumerate(pg.bundle_specs)}, "strategy": pg.strategy, "state": "CREATED"}


def remove_placement_group(pg) -> None:
    return None
