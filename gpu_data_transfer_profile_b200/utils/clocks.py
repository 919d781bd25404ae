"""Samples SM clocks and throttle reasons with `nvidia-smi` while a timed region runs.
Read-only: nothing here changes a GPU setting."""
from __future__ import annotations

import shutil
import statistics
import subprocess
import tempfile
from typing import Optional

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
           "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.out = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        self.out = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = subprocess.Popen(
            [exe, f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
             "-lms", str(self.period_ms)], stdout=self.out, stderr=subprocess.DEVNULL)
        return self

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.flush()
        self.out.seek(0)
        return parse_clock_csv(self.out.read())


def parse_clock_csv(text: str) -> dict:
    sm, mx, pw, reasons = [], [], [], set()
    names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
    for line in text.strip().splitlines():
        p = [x.strip() for x in line.split(",")]
        if len(p) < 9:
            continue
        try:
            sm.append(float(p[1]))
            mx.append(float(p[2]))
            pw.append(float(p[3]))
        except ValueError:
            continue
        for name, v in zip(names, p[5:9]):
            if v.lower().startswith("active"):
                reasons.add(name)
    if not sm:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    # samples under load: the upper half by power draw
    order = sorted(range(len(sm)), key=lambda i: pw[i])
    load = [sm[i] for i in order[len(order) // 2:]]
    return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
            "samples": len(sm), "power_w_max": max(pw)}
