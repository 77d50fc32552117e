"""SM clock and throttle reasons of a GPU sampled while a timed region runs.

A power-capped B200 settles at different SM clocks on different boxes and workloads (1.50-1.62 GHz in the
measured training steps), so an iteration time is only comparable with the clock it ran at.  ``ClockSampler``
reads them with ``nvidia-smi`` (reading only; no setting of the GPU is touched) every 200 ms in a helper
process and summarises the samples: median SM clock, maximum clock, peak power and the throttle reasons seen.
The exec entry point stores the summary of rank 0's GPU beside the measured latency
(``exec_clocks`` in ``summary.json``).
"""
from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Dict, List

QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
REASONS = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]


def summarise(lines: List[str]) -> Dict:
    """Summary of ``nvidia-smi --format=csv,noheader,nounits`` lines for ``QUERY``."""
    sm, mx, power, reasons = [], [], [], set()
    for ln in lines:
        parts = [p.strip() for p in ln.split(",")]
        if len(parts) < 9:
            continue
        try:
            sm.append(float(parts[1]))
            mx.append(float(parts[2]))
            power.append(float(parts[3]))
        except ValueError:
            continue
        for name, val in zip(REASONS, parts[5:9]):
            if val.lower().startswith("active"):
                reasons.add(name)
    return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


class ClockSampler:
    def __init__(self, index: int, period_ms: int = 200, executable: str = "nvidia-smi"):
        self.index, self.period_ms, self.executable = int(index), int(period_ms), executable
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                [self.executable, f"--id={self.index}", f"--query-gpu={QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> Dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [f"{self.executable} unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        return summarise(self.lines)
