"""Locates, (re)builds if necessary, and loads the native extension ``_C.so``.

The reference loads ``lib<package>.so`` from the package's parent directory and prints the path
on import (torch_dist_ext/__init__.py:8-12). Here the library sits inside the package, the
import is silent, and a missing or unloadable library is an error - there is no Python
fallback for the kernels.
"""
from __future__ import annotations

import logging
import os
from pathlib import Path

import torch

log = logging.getLogger("torch_dist_ext_b200")

# TDX_BOUNDS=1 selects the range-checking flavour (built by `python -m torch_dist_ext_b200._build --bounds`):
# same ops, but every store of the fused all-reduce kernels into a symmetric allocation is checked
# against the allocation's extent and a violation becomes a status code instead of a stray write.
_CHECKED = os.environ.get("TDX_BOUNDS", "0") not in ("0", "", "false", "off")
# TDX_TRACE=1 selects the tracing flavour (`--trace`): the fused all-reduce kernels record when each block
# passed each phase of its protocol (utils/tracing.py: PhaseTrace reads the record).
_TRACED = not _CHECKED and os.environ.get("TDX_TRACE", "0") not in ("0", "", "false", "off")
_LIB = Path(__file__).resolve().parent / ("_C_bounds.so" if _CHECKED else "_C_trace.so" if _TRACED else "_C.so")
_loaded = False


def lib_path() -> Path:
    return _LIB


def load() -> None:
    """Load the extension once. Builds it first when it does not exist and nvcc is present."""
    global _loaded
    if _loaded:
        return
    if not _LIB.exists() or os.environ.get("TDX_REBUILD") == "1":
        from . import _build

        log.info("building native extension (first use)")
        _build.build(checked=_CHECKED, traced=_TRACED)
    try:
        torch.ops.load_library(str(_LIB))
    except OSError as e:  # pragma: no cover - depends on the machine
        raise ImportError(
            f"torch_dist_ext_b200: could not load {_LIB}: {e}. Rebuild with "
            f"`python -m torch_dist_ext_b200._build --force`.") from e
    _loaded = True
    log.debug("loaded %s", _LIB)


def ops():
    load()
    return torch.ops.torch_dist_ext


def classes():
    load()
    return torch.classes.torch_dist_ext
