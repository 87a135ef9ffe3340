"""NVTX ranges around the library's calls, behind a flag.

The reference has no tracing in the library (its test wraps one call in ``torch.profiler``,
test/test_all_reduce_fusion.py:50-66). Here ``TDX_NVTX=1`` (or ``enable(True)``) makes every
public op and every decoder layer open an NVTX range, so that a timeline profiler shows which
launches belong to which call; when off, the cost is one attribute test per call.
"""
from __future__ import annotations

import functools
import os

_enabled = os.environ.get("TDX_NVTX", "0") not in ("0", "", "false", "off")
_push = _pop = None


def _bind():
    global _push, _pop
    if _push is None:
        import torch

        _push, _pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop


def enable(on: bool = True) -> None:
    """Switch the ranges on or off at run time."""
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


def set_backend(push, pop) -> None:
    """Replace the functions that open and close a range (tests record the calls with it)."""
    global _push, _pop
    _push, _pop = push, pop


class _Range:
    __slots__ = ("name",)

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        _bind()
        _push(self.name)

    def __exit__(self, *exc):
        _pop()
        return False


class _Off:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_OFF = _Off()


def nvtx_range(name: str):
    """Context manager: an NVTX range called ``name`` when tracing is on, nothing otherwise."""
    return _Range(name) if _enabled else _OFF


def traced(name: str):
    """Decorator: run the function inside an NVTX range called ``name`` when tracing is on."""

    def wrap(fn):
        @functools.wraps(fn)
        def inner(*args, **kwargs):
            if not _enabled:
                return fn(*args, **kwargs)
            _bind()
            _push(name)
            try:
                return fn(*args, **kwargs)
            finally:
                _pop()

        return inner

    return wrap


# ---- phase time stamps of the fused all-reduce kernels (tracing flavour of the library) --------------------

TRACE_SLOTS = 16
TRACE_MAX_BLOCKS = 1024
TRACE_PHASES = {2: "pushed", 3: "cleared", 4: "gathered", 5: "owner_done", 6: "trailer", 7: "received", 8: "end"}


class PhaseTrace:
    """Where the time of one fused all-reduce call goes, block by block.

    The tracing flavour of the library (built with ``python -m torch_dist_ext_b200._build --trace``, loaded when
    ``TDX_TRACE=1``) makes thread 0 of every block record a clock value as it passes each phase of the
    protocol: rows pushed, previous buffer cleared, peers' vectors gathered, finished row pushed by its owner,
    trailer and data of a received row arrived, end. This class owns the device buffer those values go to and
    turns it into microseconds since the block started (``summary``). The reference has nothing comparable; its
    only timing aid is the profiler table its test prints (test/test_all_reduce_fusion.py:50-66).

    The release flavour ignores the buffer, so ``summary`` then reports no phases.
    """

    def __init__(self, comm_process):
        import torch

        self._comm = comm_process
        self.buf = torch.zeros(TRACE_MAX_BLOCKS * TRACE_SLOTS, dtype=torch.int64, device=comm_process.device)
        comm_process.comm.set_trace(self.buf)

    def clear(self) -> None:
        self.buf.zero_()

    def close(self) -> None:
        self._comm.comm.set_trace(None)

    def summary(self) -> dict:
        """Per phase: minimum / median / maximum over the blocks of the last traced call, in microseconds since the
        block's own start; ``start_spread_us`` and ``span_us`` place the blocks against each other (global timer)."""
        import torch

        torch.cuda.synchronize(self.buf.device)
        t = self.buf.cpu().view(TRACE_MAX_BLOCKS, TRACE_SLOTS)
        return summarize_trace(t)


def summarize_trace(t) -> dict:
    """``t``: int64 ``[blocks, 16]`` as written by the kernels (rows of zeros = blocks that did not run)."""
    import torch

    live = t[:, 0] != 0
    t = t[live]
    if t.shape[0] == 0:
        return {"blocks": 0, "phases": {}}
    start_ns, start_clk, end_clk, end_ns = t[:, 0], t[:, 1], t[:, 8], t[:, 9]
    dur_ns = (end_ns - start_ns).double().clamp_min(1)
    dur_clk = (end_clk - start_clk).double().clamp_min(1)
    ghz = float((dur_clk / dur_ns).median())         # SM clock as the blocks saw it
    out = {"blocks": int(t.shape[0]), "sm_clock_ghz": round(ghz, 3),
           "start_spread_us": round(float(start_ns.max() - start_ns.min()) / 1e3, 2),
           "span_us": round(float(end_ns.max() - start_ns.min()) / 1e3, 2), "phases": {}}
    for slot, name in TRACE_PHASES.items():
        seen = t[:, slot] != 0
        if not bool(seen.any()):
            continue
        us = (t[seen, slot] - t[seen, 1]).double() / ghz / 1e3
        out["phases"][name] = {"blocks": int(seen.sum()), "min_us": round(float(us.min()), 2),
                               "median_us": round(float(us.median()), 2), "max_us": round(float(us.max()), 2)}
    return out
