"""Device-side timing helpers shared by bench.py, the benchmarks and the tests.

The reference's only timing facility is a torch.profiler table printed by its Python test
(test/test_all_reduce_fusion.py:50-66). These helpers time with CUDA events on the launching
stream, defeat L2 reuse between iterations, and sample the SM clock and throttle reasons while
the timed region runs.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Callable, List, Optional

import torch


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so that the next kernel starts cold."""

    def __init__(self, device=None, nbytes: int = 256 << 20):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device or "cuda")

    def __call__(self) -> None:
        self.buf.zero_()


def cuda_time_ms(fn: Callable[[], None], iters: int, warmup: int = 3,
                 flush: Optional[L2Flusher] = None) -> List[float]:
    """Per-iteration device time of ``fn`` in milliseconds (CUDA events, current stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush is not None:
            flush()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        out.append(a.elapsed_time(b))
    return out


_QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
          "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
          "clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples nvidia-smi clocks for one GPU in a background thread (read-only queries)."""

    def __init__(self, index: int = 0, period_s: float = 0.2):
        self.index, self.period = index, period_s
        self.samples: List[List[str]] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=10)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }
