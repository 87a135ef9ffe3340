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
