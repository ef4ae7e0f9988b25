"""Device-side timing helpers shared by the benchmarks.

Every number is taken with CUDA events on the launching stream after warm-up, with an L2 flush (a
write larger than the 126 MB L2) between timed iterations when the operands are smaller than L2, and
multi-GPU results are the maximum over ranks.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
import time

import torch

_FLUSH = {}


def l2_flush(device=None):
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    buf = _FLUSH.get(dev)
    if buf is None:
        buf = _FLUSH[dev] = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    buf.zero_()


def time_cuda(fn, iters: int = 10, warmup: int = 3, flush: bool = True, barrier=None):
    """Median and minimum milliseconds of fn() over `iters` runs.

    Per iteration: ranks meet (host barrier), the L2 flush is queued, then start event, fn(), stop event.  The flush
    keeps the GPU busy while the host enqueues fn, so the interval between the events is device time of fn, not the
    host's launch path; it also makes every iteration start from a cold L2.
    """
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if barrier is not None:
            barrier()
        if flush:
            l2_flush()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times), min(times)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu, self.period = gpu_index, period_ms
        self.rows, self._proc, self._thread = [], None, None

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period),
                                           "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._read, daemon=True)
            self._thread.start()
        except OSError:
            self._proc = None
        return self

    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self._proc:
            time.sleep(self.period / 1000.0)
            self._proc.terminate()
            try:
                self._proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        return False

    def summary(self) -> dict:
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx = max(mx, float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}
