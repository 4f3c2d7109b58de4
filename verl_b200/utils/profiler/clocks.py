"""Read-only sampling of a GPU's SM clock and throttle reasons while a timed region runs.

A timing is only worth quoting with the clocks it was taken at: a thermal or hardware slowdown, or a clock left locked
low by someone else, makes it meaningless. The sampler reads through NVML in a thread of this process (a few samples even
for a region of tens of milliseconds); when NVML cannot be loaded it falls back to an ``nvidia-smi`` subprocess. It changes
no setting of the GPU.
"""

from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Optional

__all__ = ["ClockSampler"]

_REASONS = {  # NVML clocks-event-reason bits that matter for a benchmark
    0x0000000000000008: "hw_slowdown",
    0x0000000000000040: "hw_thermal_slowdown",
    0x0000000000000020: "sw_thermal_slowdown",
    0x0000000000000004: "sw_power_cap",
}
_SMI_Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
          "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """``start()`` ... timed region ... ``stop()`` -> ``{"sm_mhz": median under load, "sm_max_mhz", "reasons": [...],
    "power_w_max", "samples"}``. ``snapshot()`` summarises the samples so far without stopping."""

    def __init__(self, index: int = 0, period_s: float = 0.02, nvml=None):
        self.index, self.period_s = int(index), float(period_s)
        self._nvml = nvml  # injectable for tests (an object with the pynvml functions used below)
        self._samples: list[tuple[float, float, int]] = []  # (sm MHz, power W, reason bits)
        self._max_mhz: Optional[float] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._proc = None
        self._lines: list[str] = []
        self.backend = "none"

    # ---- NVML
    def _nvml_open(self):
        nv = self._nvml
        if nv is None:
            import pynvml as nv  # provided by nvidia-ml-py
        nv.nvmlInit()
        h = nv.nvmlDeviceGetHandleByIndex(self._physical_index())
        self._max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        return nv, h

    def _physical_index(self) -> int:
        import os

        vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        ids = [x for x in vis.split(",") if x.strip() != ""]
        if ids and self.index < len(ids) and ids[self.index].strip().isdigit():
            return int(ids[self.index])
        return self.index

    def _nvml_loop(self, nv, h):
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(h) / 1e3
                except Exception:
                    watts = 0.0
                self._samples.append((mhz, watts, int(get_reasons(h))))
            except Exception:
                pass
            self._stop.wait(self.period_s)

    # ---- nvidia-smi fallback
    def _smi_read(self):
        for ln in self._proc.stdout:
            self._lines.append(ln.strip())

    def start(self) -> "ClockSampler":
        try:
            nv, h = self._nvml_open()
            self.backend = "nvml"
            self._thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
            self._thread.start()
            return self
        except Exception:
            pass
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={_SMI_Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                           "-i", str(self._physical_index())], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.backend = "nvidia-smi"
            threading.Thread(target=self._smi_read, daemon=True).start()
        except Exception:
            self._proc = None
        return self

    def snapshot(self) -> dict:
        if self.backend == "nvml":
            samples = list(self._samples)
            # "under load": samples at or above 60 % of the highest clock seen (idle samples before / after do not count)
            top = max((s[0] for s in samples), default=0.0)
            busy = [s[0] for s in samples if s[0] >= 0.6 * top and s[0] > 0]
            bits = 0
            for s in samples:
                bits |= s[2]
            return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": self._max_mhz,
                    "reasons": sorted(name for bit, name in _REASONS.items() if bits & bit),
                    "power_w_max": round(max((s[1] for s in samples), default=0.0), 1), "samples": len(samples)}
        if self.backend == "nvidia-smi":
            sm, mx, watts, reasons = [], [], [], set()
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for ln in list(self._lines):
                f = [x.strip() for x in ln.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                    watts.append(float(f[3]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            busy = [c for c in sm if c > 0]
            return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                    "reasons": sorted(reasons), "power_w_max": max(watts) if watts else None, "samples": len(sm)}
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"], "samples": 0}

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
        if self._proc is not None:
            time.sleep(0.05)
            self._proc.terminate()
        return self.snapshot()

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.result = self.stop()
        return False
