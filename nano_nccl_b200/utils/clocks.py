"""Samples SM clocks, power and throttle reasons of one GPU while a timed region runs.

Reads only (NVML queries through the nvidia-ml-py binding, every few milliseconds, from a thread);
falls back to an `nvidia-smi -lms` subprocess when the binding is unavailable. Nothing is ever set.
"""
import subprocess
import threading
import time


class ClockSampler:
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index, period_s=0.004):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.rows = []  # (wall time, sm MHz, max sm MHz, watts, reasons bitmask)
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None
        self.source = "none"

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self._max = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
            self.source = "nvml"
        except Exception:
            self._nvml = None
            self.source = "nvidia-smi"
        self._thread = threading.Thread(target=self._run_nvml if self._nvml else self._run_smi, daemon=True)
        self._thread.start()

    def _run_nvml(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                clk = n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)
                try:
                    watts = n.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                except Exception:
                    watts = 0.0
                try:
                    reasons = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                except Exception:
                    reasons = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                self.rows.append((time.time(), float(clk), float(self._max), watts, int(reasons)))
            except Exception:
                pass
            time.sleep(self.period_s)

    def _run_smi(self):
        query = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={query}", "--format=csv,noheader,nounits", "-lms", "50"],
                                    stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            return
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            line = proc.stdout.readline()
            if not line:
                break
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8 or parts[0] != str(self.gpu_index):
                continue
            try:
                mask = 0
                for name, val in zip(names, parts[4:8]):
                    if val.lower().startswith("active"):
                        mask |= self.REASONS[name]
                self.rows.append((time.time(), float(parts[1]), float(parts[2]), float(parts[3] or 0), mask))
            except ValueError:
                continue
        proc.terminate()

    def stop(self, window=None):
        """Summary dict. ``window=(t0, t1)`` (wall-clock seconds) keeps the samples taken inside the
        timed region; when none fell inside, all samples of the run are used and ``scope`` says so."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        inside = [r for r in self.rows if window and window[0] <= r[0] <= window[1]]
        scope = "timed region"
        if not inside:
            inside, scope = self.rows, "whole run (no sample fell inside the timed region)"
        clocks = sorted(r[1] for r in inside)
        mask = 0
        for r in inside:
            mask |= r[4]
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max((r[2] for r in inside), default=None),
                "power_w_max": round(max((r[3] for r in inside), default=0.0), 1),
                "reasons": sorted(n for n, bit in self.REASONS.items() if mask & bit),
                "samples": len(inside), "scope": scope, "source": self.source}
