"""Host-side fault injection for health-monitoring tests.

``PIPER_FAULT="bwd:<iteration>:<dp_rank>[:sleep:<seconds>]"`` makes the
matching data-parallel rank raise (or sleep) right before it launches the
first backward task of the given iteration, once per process (format and
latch semantics of ``src/executors.py:19-48``).  The failure is always
produced on the host, before any kernel of that task is enqueued; nothing
here makes a GPU fault.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Optional


class InjectedFault(RuntimeError):
    """Raised by the fault injector."""


@dataclass
class FaultSpec:
    point: str
    iteration: int
    dp_rank: int
    action: str = "raise"
    seconds: float = 0.0


def parse_fault_spec(text: Optional[str]) -> Optional[FaultSpec]:
    if not text:
        return None
    parts = text.split(":")
    if len(parts) < 3 or parts[0] != "bwd":
        raise ValueError(f"PIPER_FAULT must look like 'bwd:<iter>:<dp_rank>[:sleep:<s>]', got {text!r}")
    spec = FaultSpec(point=parts[0], iteration=int(parts[1]), dp_rank=int(parts[2]))
    if len(parts) >= 5 and parts[3] == "sleep":
        spec.action, spec.seconds = "sleep", float(parts[4])
    elif len(parts) > 3:
        raise ValueError(f"unsupported PIPER_FAULT action in {text!r}")
    return spec


class FaultInjector:
    def __init__(self, dp_rank: int, spec: Optional[FaultSpec] = None) -> None:
        self.dp_rank = dp_rank
        self.spec = spec if spec is not None else parse_fault_spec(os.environ.get("PIPER_FAULT"))
        self.fired = False

    def maybe_fire(self, point: str, iteration: int) -> None:
        s = self.spec
        if s is None or self.fired or s.point != point or s.iteration != iteration or s.dp_rank != self.dp_rank:
            return
        self.fired = True
        if s.action == "sleep":
            time.sleep(s.seconds)
            return
        raise InjectedFault(f"PIPER_FAULT fired at {point} iteration {iteration} dp_rank {self.dp_rank}")
