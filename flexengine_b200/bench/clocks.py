"""What a number is measured against and under: the peaks of this machine, and its clocks during the timed region."""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import threading
import time

from .shapes import FALLBACK_PEAKS


def load_peaks(path: str | None):
    """({"hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"}, "measured" | "fallback"): from the file of measured
    peaks when there is one (``path``, else ``$FLEXENGINE_PEAKS``, else ``MEASURED_PEAKS.json`` in the working
    directory), else the fallback figures."""
    for candidate in (path, os.environ.get("FLEXENGINE_PEAKS"), os.path.join(os.getcwd(), "MEASURED_PEAKS.json")):
        if not candidate or not os.path.isfile(candidate):
            continue
        try:
            with open(candidate) as f:
                data = json.load(f)
        except (OSError, ValueError):
            continue
        flat = {}

        def walk(d):
            for k, v in d.items():
                if isinstance(v, dict):
                    walk(v)
                elif isinstance(v, (int, float)) and not isinstance(v, bool):
                    flat.setdefault(k, float(v))
        walk(data)
        if "hbm_gbs" in flat and "bf16_tflops" in flat:
            flat.setdefault("bf16_tflops_sustained", flat["bf16_tflops"])
            return flat, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi (reading only) while timed regions run."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return self

        def pump():
            for line in self.proc.stdout:
                self.samples.append((time.time(), [p.strip() for p in line.split(",")]))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        return self

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        """Median SM clock and the reasons seen inside ``windows`` [(wall start, wall end)] (all samples if none fell inside)."""
        picked = [s for t, s in self.samples if any(a <= t <= b for a, b in windows)] or [s for _, s in self.samples]
        clocks, reasons, max_mhz = [], set(), None
        for s in picked:
            try:
                clocks.append(float(s[0]))
                max_mhz = float(s[1])
            except (ValueError, IndexError):
                continue
            for name, value in zip(self.REASONS, s[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_mhz,
                "reasons": sorted(reasons), "samples": len(picked)}
