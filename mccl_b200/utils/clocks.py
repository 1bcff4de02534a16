"""Samples SM clocks and throttle reasons with nvidia-smi while a benchmark runs.

Read-only: nothing here changes a GPU setting.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Dict, List

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.rows: List[List[str]] = []
        self.proc = None
        self.thread = None

    def start(self) -> "ClockSampler":
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                 "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return self

        def pump():
            for line in self.proc.stdout:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) >= 9:
                    self.rows.append(parts)
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        return self

    def stop(self) -> Dict:
        if self.proc is not None:
            self.proc.terminate()   # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm = [float(r[1]) for r in self.rows if r[1].replace(".", "", 1).isdigit()]
        mx = [float(r[2]) for r in self.rows if r[2].replace(".", "", 1).isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples": len(self.rows),
        }
