class PlacementGroupSchedulingStrategy:
    def __init__(self, placement_group=None, placement_group_bundle_index: int = -1,
                 placement_group_capture_child_tasks=None) -> None:
        self.placement_group = placement_group
        self.placement_group_bundle_index = placement_group_bundle_index
        self.placement_group_capture_child_tasks = placement_group_capture_child_tasks


class NodeAffinitySchedulingStrategy:
    def __init__(self, node_id=None, soft: bool = False) -> None:
        self.node_id, self.soft = node_id, soft
