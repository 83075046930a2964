"""Plan decomposition: the global training DAG -> one DAG per device set.

SEND and RECV nodes of a pipeline boundary are deliberately not connected, so
after the directive rewrites the global DAG falls apart into connected
components, one per placement.  Each must be device-homogeneous and the
device sets distinct; components are returned sorted by device tuple, and
the index in that list is the physical pipeline rank
(``src/piper.py:84-165`` defines the same contract).
"""
from __future__ import annotations

from .dag import TrainingDAG


def split_by_device_set(dag: TrainingDAG) -> list[TrainingDAG]:
    comp_of: dict[str, int] = {}
    comps: list[list[str]] = []
    for uid in dag.nodes:
        if uid in comp_of:
            continue
        cid = len(comps)
        members = [uid]
        comp_of[uid] = cid
        stack = [uid]
        while stack:
            cur = stack.pop()
            for nb in sorted(dag.succs[cur] | dag.preds[cur]):
                if nb not in comp_of:
                    comp_of[nb] = cid
                    members.append(nb)
                    stack.append(nb)
        comps.append(members)

    keyed: list[tuple[tuple, list[str]]] = []
    for ci, members in enumerate(comps):
        keys = {dag.nodes[u].device_key for u in members if dag.nodes[u].device is not None}
        if not keys:
            raise ValueError(f"component[{ci}] has no device assignment after P2P split")
        if len(keys) != 1:
            raise ValueError(f"component[{ci}] is not device-homogeneous; device sets present: {sorted(keys)}")
        keyed.append((keys.pop(), members))
    dev_keys = [k for k, _ in keyed]
    if len(set(dev_keys)) != len(dev_keys):
        raise ValueError(f"expected distinct device sets across split components, got {dev_keys}")
    keyed.sort(key=lambda kv: kv[0])
    order = {u: i for i, u in enumerate(dag.nodes)}
    return [dag.copy_subgraph(sorted(members, key=order.get)) for _, members in keyed]


_split_global_training_dag_by_pp_rank = split_by_device_set
