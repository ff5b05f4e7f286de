"""Device-side timing helpers: CUDA-event timing with L2 flush, max over ranks, clock sampling.

The reference times with per-iteration CUDA events and prints rank 0's mean
(tests/test_teramoe_performance.py:127-164); here every multi-rank number is the maximum over ranks.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

_L2_FLUSH = None


def flush_l2() -> None:
    """Overwrite a buffer larger than the 126 MB L2 so the next kernel starts from HBM."""
    global _L2_FLUSH
    if _L2_FLUSH is None:
        _L2_FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _L2_FLUSH.zero_()


def bench_cuda(fn: Callable[[], None], steps: int, warmup: int, flush: bool = True) -> List[float]:
    """Per-iteration milliseconds of fn(), CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(steps):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e))
    return times


def max_over_ranks(value: float, group=None) -> float:
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda" if torch.cuda.is_available() and dist.get_backend(group) == "nccl" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs (read-only)."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 50):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.lines: List[str] = []
        self._thread: Optional[threading.Thread] = None

    def start(self) -> "ClockSampler":
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return self

        def reader():
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self._thread = threading.Thread(target=reader, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:  # pragma: no cover
            self.proc.kill()
        if self._thread is not None:
            self._thread.join(timeout=2)
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # "under load" = samples in the upper half of the observed power range
        if sm:
            thr = (max(power) + min(power)) / 2 if power else 0
            loaded = [c for c, p in zip(sm, power) if p >= thr] or sm
            return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                    "power_w_max": max(power)}
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": sorted(reasons), "samples": 0}
