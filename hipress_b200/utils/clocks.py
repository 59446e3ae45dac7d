"""Sample SM clocks and throttle reasons with ``nvidia-smi`` while a timed region runs.

Read-only: nothing here changes a clock, a power limit or any other GPU setting.

``nvidia-smi`` needs a moment to start (longer when eight ranks start one each), and a timed
region of a few hundred milliseconds can be over before its first sample.  So the sampler is
started ahead of the region (during the warm-up steps, which run the same load), every sample
carries ``nvidia-smi``'s own timestamp, and ``mark_start()`` / ``mark_end()`` delimit the
region: ``summary()`` reports the samples inside the marks, or -- if none fell inside -- all
samples taken under load since the start, and says which.
"""
from __future__ import annotations

import datetime
import shutil
import statistics
import subprocess
import tempfile
import time
from typing import Dict, List, Optional

QUERY = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """``with ClockSampler(device_index) as c: ...`` then ``c.summary()``."""

    def __init__(self, device_index: int = 0, period_ms: int = 50):
        self.device_index = device_index
        self.period_ms = period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.file = None
        self.t_start: Optional[float] = None
        self.t_end: Optional[float] = None

    def mark_start(self) -> None:
        self.t_start = time.time()

    def mark_end(self) -> None:
        self.t_end = time.time()

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

    @staticmethod
    def _stamp(text: str) -> Optional[float]:
        try:
            return datetime.datetime.strptime(text, "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def summary(self) -> Dict:
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        samples = []
        for r in self.rows():
            if len(r) < 10:
                continue
            try:
                sm, mx = float(r[2]), float(r[3])
            except ValueError:
                continue
            active = [name for name, val in zip(names, r[6:10]) if val.lower().startswith("active")]
            samples.append((self._stamp(r[0]), sm, mx, active))
        if not samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "window": "no samples"}
        window = "timed region"
        inside = samples
        if self.t_start is not None and self.t_end is not None:
            inside = [x for x in samples if x[0] is not None and self.t_start <= x[0] <= self.t_end]
            if not inside:
                inside, window = samples, "warm-up and timed region (no sample fell inside the timed region)"
        reasons = sorted({name for x in inside for name in x[3]})
        return {"sm_mhz": statistics.median(x[1] for x in inside), "sm_max_mhz": max(x[2] for x in inside),
                "reasons": reasons, "samples": len(inside), "window": window}
