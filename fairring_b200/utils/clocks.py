"""Samples SM clocks and clock-event (throttle) reasons while a benchmark runs.

Only reads NVML counters; nothing is ever set.
"""

from __future__ import annotations

import statistics
import threading
import time


class ClockSampler:
    def __init__(self, device_index: int = 0, period_s: float = 0.2):
        self.device_index = device_index
        self.period_s = period_s
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self.power_w_max = 0.0
        self._stop = threading.Event()
        self._thread = None
        self._ok = False
        try:
            import pynvml

            self._nvml = pynvml
            pynvml.nvmlInit()
            self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._ok = True
        except Exception:  # no NVML (CPU box): report nothing rather than fail
            self._ok = False

    _REASONS = {
        "hw_slowdown": 0x8,
        "sw_power_cap": 0x4,
        "sw_thermal_slowdown": 0x20,
        "hw_thermal_slowdown": 0x40,
        "hw_power_brake_slowdown": 0x80,
    }

    def _loop(self) -> None:
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(int(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
                try:
                    mask = int(n.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for name, bit in self._REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
                self.power_w_max = max(self.power_w_max, n.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            except Exception:
                pass
            time.sleep(self.period_s)

    def __enter__(self):
        if self._ok:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        if not self._ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {
            "sm_mhz": int(statistics.median(self.samples)),
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
            "power_w_max": round(self.power_w_max, 1),
        }
