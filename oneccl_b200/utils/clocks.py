"""Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
from __future__ import annotations

import shutil
import statistics
import subprocess
import threading
import time

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Context manager: starts one ``nvidia-smi -lms`` for a GPU index or a list of indices (an empty
    list samples nothing: in a multi-process job one rank watches every GPU), parses the rows on exit."""

    def __init__(self, gpu_index=0, period_ms: int = 200):
        self.gpu_index = [gpu_index] if isinstance(gpu_index, int) else list(gpu_index)
        self.period_ms = period_ms
        self.rows = []  # (arrival time, csv line)
        self._windows = []  # [begin, end] pairs of time.monotonic(); empty = everything counts
        self._proc = None
        self._thread = None

    def __enter__(self):
        exe = shutil.which("nvidia-smi")
        if exe is None or not self.gpu_index:
            return self
        try:
            self._proc = subprocess.Popen(
                [exe, f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", ",".join(str(i) for i in self.gpu_index),
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self

        def pump():
            for line in self._proc.stdout:
                self.rows.append((time.monotonic(), line.strip()))

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._proc is not None and self._proc.poll() is None:
            self._proc.terminate()  # the exact child started above
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            if self._thread is not None:
                self._thread.join(timeout=2)
        return False

    def begin(self):
        """Opens a window: only samples that arrive inside windows are summarised (the tool takes a
        few hundred ms to start, so it is launched well before the region of interest)."""
        self._windows.append([time.monotonic(), None])

    def end(self):
        if self._windows and self._windows[-1][1] is None:
            self._windows[-1][1] = time.monotonic()

    def _inside(self, t: float) -> bool:
        if not self._windows:
            return True
        return any(b <= t <= (e if e is not None else float("inf")) for b, e in self._windows)

    def summary(self) -> dict:
        sm, mx, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, row in self.rows:
            if not self._inside(t):
                continue
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "reasons": sorted(reasons), "samples": len(sm)}
