"""Sample SM clocks and throttle reasons with nvidia-smi while a benchmark runs (read-only)."""

from __future__ import annotations

import statistics
import subprocess
import threading

_QUERY = (
    "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
    "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
    "clocks_event_reasons.sw_power_cap"
)
_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")


class ClockSampler:
    """``with ClockSampler(gpu_index) as cs: ...; cs.summary()``."""

    def __init__(self, index: int = 0, period_ms: int = 100):
        self.index, self.period_ms = index, period_ms
        self.samples: list[tuple[float, float, float, tuple[bool, ...]]] = []
        self._proc = None
        self._thread = None

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
        except OSError:
            self._proc = None
            return self
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()
        return self

    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm, mx, pw = float(parts[0]), float(parts[1]), float(parts[2])
            except ValueError:
                continue
            self.samples.append((sm, mx, pw, tuple(p.lower() == "active" for p in parts[3:7])))

    def __exit__(self, *exc):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        if self._thread is not None:
            self._thread.join(timeout=5)
        return False

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = [name for i, name in enumerate(_REASONS) if any(s[3][i] for s in self.samples)]
        return {
            "sm_mhz": statistics.median(s[0] for s in self.samples),
            "sm_max_mhz": max(s[1] for s in self.samples),
            "power_w_max": max(s[2] for s in self.samples),
            "reasons": reasons,
            "samples": len(self.samples),
        }
