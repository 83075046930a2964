"""Merging per-rank ``torch.profiler`` traces into one Chrome trace per data-parallel rank.

Each rank exports ``dp{d}_pp{p}.json``.  The merger gives every rank its own pid block, prefixes process
names with the rank, and renames GPU kernels to ``<dag label>::<kernel>`` by joining the CPU
``record_function`` range of a DAG node (label ``TASK:tags:uid...``) with the GPU events launched inside it
through their ``External id`` (what ``examples/test_harness.py:258-521`` of the reference does for Ray actors).
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Optional

_LABEL = re.compile(r"^[A-Z_]+:.*:uid")


def _load(path: str) -> list:
    with open(path, encoding="utf-8") as f:
        data = json.load(f)
    return data["traceEvents"] if isinstance(data, dict) else data


def relabel_gpu_events(events: list) -> int:
    """Prefix GPU events with the label of the DAG node whose CPU range launched them; returns #renamed."""
    ranges = sorted(((e["ts"], e["ts"] + e.get("dur", 0), e["name"], e.get("tid")) for e in events
                     if e.get("ph") == "X" and e.get("cat") in ("user_annotation", "cpu_op")
                     and _LABEL.match(str(e.get("name", "")))), key=lambda r: r[0])
    if not ranges:
        return 0
    launches = {}
    for e in events:
        if e.get("ph") == "X" and e.get("cat") in ("cuda_runtime", "cuda_driver"):
            ext = (e.get("args") or {}).get("External id", (e.get("args") or {}).get("correlation"))
            if ext is None:
                continue
            ts = e["ts"]
            label = next((r[2] for r in ranges if r[0] <= ts <= r[1] and (r[3] is None or r[3] == e.get("tid"))), None)
            if label:
                launches[ext] = label
    n = 0
    for e in events:
        if e.get("ph") == "X" and e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset"):
            ext = (e.get("args") or {}).get("External id", (e.get("args") or {}).get("correlation"))
            label = launches.get(ext)
            if label and "::" not in str(e.get("name")):
                e["name"] = f"{label}::{e['name']}"
                n += 1
    return n


def combine_profiles(profile_dir: str, out_dir: str, schedule: str, pp, mbs) -> list[str]:
    by_dp: dict[int, list[str]] = {}
    for path in sorted(glob.glob(os.path.join(profile_dir, "dp*_pp*.json"))):
        m = re.search(r"dp(\d+)_pp(\d+)\.json$", path)
        if m:
            by_dp.setdefault(int(m.group(1)), []).append(path)
    outputs = []
    for dp, paths in sorted(by_dp.items()):
        merged = []
        for idx, path in enumerate(paths):
            events = _load(path)
            relabel_gpu_events(events)
            ppr = int(re.search(r"_pp(\d+)\.json$", path).group(1))
            for e in events:
                if isinstance(e.get("pid"), int):
                    e["pid"] = e["pid"] + (idx + 1) * 1_000_000
                elif "pid" in e:
                    e["pid"] = f"pp{ppr}:{e['pid']}"
                if e.get("ph") == "M" and e.get("name") == "process_name":
                    e.setdefault("args", {})["name"] = f"pp{ppr} " + str(e["args"].get("name", ""))
            merged.extend(events)
        dp_count = len(by_dp)
        out = os.path.join(out_dir, f"pytorch_profile_{schedule}_pp{pp}_dp{dp_count}_mbs{mbs}_dprank{dp}.json")
        with open(out, "w", encoding="utf-8") as f:
            json.dump({"traceEvents": merged}, f)
        outputs.append(out)
    return outputs
