"""Samples SM clocks and throttle reasons while a benchmark runs (read-only: nothing here changes
a GPU setting). Uses NVML through ``pynvml`` from a background thread (a sample every few
milliseconds); falls back to polling ``nvidia-smi`` when NVML cannot be loaded."""
from __future__ import annotations

import shutil
import statistics
import subprocess
import threading
import time

_SMI_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: float = 5.0):
        self.gpu_index = gpu_index
        self.period_s = period_ms / 1000.0
        self.samples: list[tuple[float, float, float, int]] = []     # (time, sm MHz, power W, reasons bitmask)
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._smi_lines: list[str] = []
        self._proc = None

    def _physical_index(self) -> int:
        import os

        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                return int(vis.split(",")[self.gpu_index])
            except (ValueError, IndexError):
                pass
        return self.gpu_index

    def start(self) -> "ClockSampler":
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self._nvml = (pynvml, h)

            def pump():
                while not self._stop.is_set():
                    try:
                        sm = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                        pw = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                        rs = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)) if hasattr(
                            pynvml, "nvmlDeviceGetCurrentClocksEventReasons") else int(
                            pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                        self.samples.append((time.perf_counter(), sm, pw, rs))
                    except Exception:
                        pass
                    time.sleep(self.period_s)

            self._thread = threading.Thread(target=pump, daemon=True)
            self._thread.start()
            return self
        except Exception:
            self._nvml = None
        exe = shutil.which("nvidia-smi")
        if exe is not None:
            self._proc = subprocess.Popen(
                [exe, f"--query-gpu={_SMI_FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self._physical_index())], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)

            def pump_smi():
                for line in self._proc.stdout:
                    self._smi_lines.append(line.strip())

            self._thread = threading.Thread(target=pump_smi, daemon=True)
            self._thread.start()
        return self

    def mark(self) -> float:
        return time.perf_counter()

    def stop(self, t_begin: float | None = None, t_end: float | None = None) -> dict:
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()          # the exact process started above
            try:
                self._proc.wait(timeout=5)
            except Exception:
                pass
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self._nvml is not None:
            pynvml, _ = self._nvml
            sel = [s for s in self.samples if (t_begin is None or s[0] >= t_begin) and (t_end is None or s[0] <= t_end)]
            if not sel:
                sel = self.samples[-3:]
            try:
                pynvml.nvmlShutdown()
            except Exception:
                pass
            if not sel:
                return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
            mask = 0
            for s in sel:
                mask |= s[3]
            names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
            return {"sm_mhz": statistics.median(s[1] for s in sel), "sm_max_mhz": self.sm_max,
                    "power_w_max": max(s[2] for s in sel), "reasons": sorted(v for k, v in names.items() if mask & k),
                    "samples": len(sel), "source": "nvml"}
        sm, mx, reasons = [], [], set()
        for ln in self._smi_lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}
