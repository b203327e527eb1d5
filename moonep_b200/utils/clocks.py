"""Sample SM clocks and throttle reasons while a benchmark runs (read-only NVML queries)."""

from __future__ import annotations

import statistics
import threading
import time

_REASON_BITS = {
    "hw_slowdown": 0x8,
    "sw_power_cap": 0x4,
    "sw_thermal_slowdown": 0x20,
    "hw_thermal_slowdown": 0x40,
}


def _physical_index(index: int) -> int:
    import os

    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v.strip() for v in vis.split(",") if v.strip()]
        if index < len(ids) and ids[index].isdigit():
            return int(ids[index])
    return index


class ClockSampler:
    """``with ClockSampler(gpu_index) as cs: ...; cs.summary()`` — samples every ``period_ms``."""

    def __init__(self, index: int = 0, period_ms: int = 10):
        self.index, self.period = _physical_index(index), period_ms / 1e3
        self.samples: list[tuple[int, int, float, int]] = []
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            # the first call of each query is the slow one (tens of milliseconds): make it before the timed region
            nv, h = pynvml, self._handle
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
            nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            nv.nvmlDeviceGetPowerUsage(h)
            try:
                nv.nvmlDeviceGetCurrentClocksEventReasons(h)
            except AttributeError:
                nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
        except Exception:  # noqa: BLE001 - sampling is best effort
            self._nvml = None
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        nv, h = self._nvml, self._handle
        while not self._stop.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
                pw = nv.nvmlDeviceGetPowerUsage(h) / 1e3
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except AttributeError:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.samples.append((sm, mx, pw, int(rs)))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return False

    def reset(self):
        """Forget the samples taken so far (e.g. those of a warm-up inside the ``with`` block)."""
        self.samples = []

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = [name for name, bit in _REASON_BITS.items() if any(s[3] & bit for s in self.samples)]
        return {
            "sm_mhz": statistics.median(s[0] for s in self.samples),
            "sm_max_mhz": max(s[1] for s in self.samples),
            "power_w_max": max(s[2] for s in self.samples),
            "reasons": reasons,
            "samples": len(self.samples),
        }
