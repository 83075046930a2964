"""Schedule-directive files: loading, shape validation and derived facts.

A schedule is a JSON array of directive objects (``place``, ``replicate``,
``shard``, ``split``, ``order``).  This module checks the shape of each
directive and derives ``{name, path, num_stages, pp_degree, dp_degree,
num_microbatches}`` from the ``place`` and ``split`` entries, with the same
rules as the reference loader (``src/schedule.py:6-99``): ``num_stages`` is
the number of distinct ``PP`` indices, ``pp_degree`` the number of distinct
device lists and ``dp_degree`` the length of a device list.
"""
from __future__ import annotations

import json
import os
from typing import Any

FILTER_OPS = ("place", "replicate", "shard", "split")


def validate_directive_shape(directive: Any, idx: int) -> None:
    if not isinstance(directive, dict):
        raise ValueError(f"schedule directive[{idx}] must be an object, got: {type(directive)}")
    op = directive.get("op")
    if op in FILTER_OPS:
        if not isinstance(directive.get("filter"), dict):
            raise ValueError(f"{op} directive[{idx}] requires object field 'filter': {directive}")
        if "filters" in directive:
            raise ValueError(f"{op} directive[{idx}] does not accept field 'filters': {directive}")
    elif op == "order":
        groups = directive.get("filters")
        if not isinstance(groups, list) or not groups:
            raise ValueError(f"order directive[{idx}] requires non-empty list field 'filters': {directive}")
        for gi, group in enumerate(groups):
            if not isinstance(group, list) or not group:
                raise ValueError(f"order directive[{idx}] group[{gi}] must be a non-empty list: {directive}")
            for fi, flt in enumerate(group):
                if not isinstance(flt, dict):
                    raise ValueError(
                        f"order directive[{idx}] group[{gi}][{fi}] must be a filter object: {directive}")
    else:
        raise ValueError(f"schedule directive[{idx}] has unsupported op: {directive}")


def load_schedule_directives(path: str) -> list[dict]:
    with open(path, "r", encoding="utf-8") as f:
        directives = json.load(f)
    if not isinstance(directives, list):
        raise ValueError(f"schedule directives file must contain a list, got: {type(directives)}")
    for i, d in enumerate(directives):
        validate_directive_shape(d, i)
        if d.get("op") == "split" and d.get("num_microbatches") == "__MBS__":
            raise ValueError("split.num_microbatches must be encoded in the schedule JSON; "
                             "'__MBS__' is no longer supported")
    return directives


def derive_schedule_info(directives: list[dict], schedule_path: str) -> dict[str, Any]:
    stage_devices: dict[int, list[int]] = {}
    n_mbs = None
    for d in directives:
        if not isinstance(d, dict):
            continue
        if d.get("op") == "place":
            flt = d.get("filter")
            pp = flt.get("PP") if isinstance(flt, dict) else None
            devices = d.get("devices", d.get("device"))
            if pp is None or not isinstance(devices, list) or not devices:
                raise ValueError(f"place directive must include PP filter and non-empty devices: {d}")
            stage_devices[int(pp)] = [int(x) for x in devices]
        elif d.get("op") == "split":
            n = int(d.get("num_microbatches", 0))
            if n <= 0:
                raise ValueError(f"split directive requires num_microbatches > 0: {d}")
            if n_mbs is not None and n_mbs != n:
                raise ValueError(f"multiple split directives disagree on num_microbatches: {n_mbs} vs {n}")
            n_mbs = n
    if not stage_devices:
        raise ValueError("schedule JSON must include place directives with PP filters")
    stages = sorted(stage_devices)
    if stages != list(range(len(stages))):
        raise ValueError(f"PP indices must be contiguous from 0, got {stages}")
    counts = {len(v) for v in stage_devices.values()}
    if len(counts) != 1:
        raise ValueError(f"all PP place directives must use the same device count, got {stage_devices}")
    if n_mbs is None:
        raise ValueError("schedule JSON must include a split directive with num_microbatches")
    return {
        "name": os.path.splitext(os.path.basename(schedule_path))[0],
        "path": schedule_path,
        "num_stages": len(stages),
        "pp_degree": len({tuple(v) for v in stage_devices.values()}),
        "dp_degree": counts.pop(),
        "num_microbatches": n_mbs,
    }


def load_schedule_info(path: str) -> dict[str, Any]:
    return derive_schedule_info(load_schedule_directives(path), path)


def stage_device_map(directives: list[dict]) -> dict[int, tuple[int, ...]]:
    """PP stage index -> device tuple (as written, order preserved)."""
    out: dict[int, tuple[int, ...]] = {}
    for d in directives:
        if isinstance(d, dict) and d.get("op") == "place":
            pp = (d.get("filter") or {}).get("PP")
            devs = d.get("devices", d.get("device"))
            if pp is not None and pp != "*" and isinstance(devs, list):
                out[int(pp)] = tuple(int(x) for x in devs)
    return out
