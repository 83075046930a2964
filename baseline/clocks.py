"""``nvidia-smi`` sampler of SM clocks and throttle reasons, shared by both arms of the benchmark."""
from __future__ import annotations

import statistics
import subprocess
import threading


class ClockSampler:
    """Samples the SM clock and the throttle reasons of the given GPUs every 200 ms while a timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, indices) -> None:
        self.indices = [int(i) for i in ([indices] if isinstance(indices, int) else indices)]
        self.rows, self.proc = [], None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", ",".join(str(i) for i in self.indices), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        return self.summarise(self.rows)

    @classmethod
    def summarise(cls, rows) -> dict:
        sm, mx, reasons = [], [], set()
        for r in rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(cls.REASONS, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}
