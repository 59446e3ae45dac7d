"""Sample SM clocks and throttle reasons with ``nvidia-smi`` while a timed region runs.

Read-only: nothing here changes a clock, a power limit or any other GPU setting.
"""
from __future__ import annotations

import shutil
import statistics
import subprocess
import tempfile
from typing import Dict, List, Optional

QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """``with ClockSampler(device_index) as c: ...`` then ``c.summary()``."""

    def __init__(self, device_index: int = 0, period_ms: int = 200):
        self.device_index = device_index
        self.period_ms = period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.file = None

    def __enter__(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = subprocess.Popen(
            [exe, f"--query-gpu={QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
             "-i", str(self.device_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()  # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def rows(self) -> List[List[str]]:
        if self.file is None:
            return []
        self.file.flush()
        with open(self.file.name) as f:
            return [[c.strip() for c in line.split(",")] for line in f if line.strip()]

    def summary(self) -> Dict:
        rows = self.rows()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}
