"""Device-side timing and clock sampling.

Multi-GPU numbers are CUDA-event durations on the launching stream, bracketed by a barrier and
a device synchronise, reduced with MAX over ranks; wall clocks are never used for throughput.
`ClockSampler` polls `nvidia-smi` in a background thread while a timed region runs and
reports the median SM clock and every throttle reason that was active.
"""

from __future__ import annotations

import statistics
import subprocess
import threading

import torch
import torch.distributed as dist


class DeviceTimer:
    """`with DeviceTimer() as t: ...` then `t.ms` (this rank) / `t.max_ms()` (max over ranks)."""

    def __init__(self, barrier=True):
        self.barrier = barrier
        self.ms = None

    def __enter__(self):
        if self.barrier and dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()
        self._a = torch.cuda.Event(enable_timing=True)
        self._b = torch.cuda.Event(enable_timing=True)
        self._a.record()
        return self

    def __exit__(self, *exc):
        self._b.record()
        torch.cuda.synchronize()
        self.ms = self._a.elapsed_time(self._b)
        if self.barrier and dist.is_initialized():
            dist.barrier()
        return False

    def max_ms(self):
        if not dist.is_initialized():
            return self.ms
        t = torch.tensor([self.ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())


_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index=0, period_s=0.2):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _poll(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits",
                     "-i", str(self.gpu_index)],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(self.period_s)

    def __enter__(self):
        self._thread = threading.Thread(target=self._poll, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
        return False

    def summary(self):
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[1]))
                mx.append(float(s[2]))
                power.append(float(s[3]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, s[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "reasons": sorted(reasons), "samples": len(sm)}
