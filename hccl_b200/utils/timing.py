"""Timing hygiene helpers: CUDA-event timing, L2 flush, nvidia-smi clock sampling
during the timed region, and nccl-tests style bus-bandwidth factors."""
from __future__ import annotations

import statistics
import subprocess
import threading

import torch


def device_time_ms(fn, iters: int, warmup: int = 3, flush_l2: bool = False) -> float:
    """Mean device time of ``fn`` over ``iters`` launches, CUDA events on the current stream."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if flush is None:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(iters):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / iters
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        fn()
        t1.record()
        torch.cuda.synchronize()
        total += t0.elapsed_time(t1)
    return total / iters


class ClockSampler:
    """Samples SM clocks and throttle reasons while a region runs (reading only; nothing is ever set).

    Reads through NVML in a thread of this process (first sample within milliseconds, so short timed regions are covered);
    falls back to an `nvidia-smi -lms` child process when the NVML binding is missing.
    """

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 20):
        self.gpu, self.period = gpu_index, period_ms
        self.samples = []          # [sm_mhz, max_mhz, watts, hw_slowdown, hw_thermal, sw_thermal, sw_power_cap] ("Active"/"Not Active")
        self._proc = None
        self._thread = None
        self._stop = threading.Event()

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu)

    def __enter__(self):
        try:
            nv, h = self._nvml_handle()
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
            bits = (0x8, 0x40, 0x20, 0x4)          # hw slowdown, hw thermal slowdown, sw thermal slowdown, sw power cap

            def poll():
                while True:
                    try:
                        r = get_reasons(h)
                        row = [str(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), str(mx),
                               str(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)]
                        row += ["Active" if r & b else "Not Active" for b in bits]
                        self.samples.append(row)
                    except Exception:
                        pass
                    if self._stop.wait(self.period / 1000.0):
                        return

            self._thread = threading.Thread(target=poll, daemon=True)
            self._thread.start()
            return self
        except Exception:
            pass
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", f"-i={self.gpu}",
                                           f"-lms={max(self.period, 100)}"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self

        def pump():
            for line in self._proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 7:
                    self.samples.append(parts)

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()          # the exact process started above
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        elif self._thread is not None:
            self._thread.join(timeout=2)
        return False

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, val in zip(self.REASONS, s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def bus_bandwidth_factor(op: str, n: int) -> float:
    """busBW = algBW * factor (nccl-tests convention)."""
    if n <= 1:
        return 1.0
    return {"all_reduce": 2.0 * (n - 1) / n, "all_gather": (n - 1) / n, "reduce_scatter": (n - 1) / n, "all_to_all": (n - 1) / n,
            "broadcast": 1.0, "reduce": 1.0}[op]
