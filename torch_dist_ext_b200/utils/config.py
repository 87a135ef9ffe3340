"""Runtime configuration.

The reference has no configuration system: its knobs are compile-time constants
(src/common/all_reduce_fusion_impl.h:17-28) and two keyword arguments of ``setup_env``
(torch_dist_ext/__init__.py:41). Here the knobs are one dataclass, overridable from the
environment:

=====================  ============================================================
``TDX_ALGO``           ``auto`` | ``oneshot`` | ``twoshot`` | ``twoshot_barrier`` |
                       ``nvls_oneshot`` | ``nvls_twoshot`` | ``oneshot_mc`` | ``twoshot_mc``
                       (the ``_mc`` forms push through ``multimem.st``: NVSwitch replicates the store)
``TDX_PDL``            ``0`` launches the fused all-reduce kernels without programmatic stream
                       serialisation (read by the native launcher)
``TDX_TIMEOUT_MS``     budget of every device-side wait (default 5000)
``TDX_LAMPORT_MB``     capacity of each of the three Lamport buffers (default 72: a 32 MiB message with its result rows)
``TDX_NVLS``           ``0`` disables the NVSwitch-multicast mapping and kernels
``TDX_WAVES``          pipeline depth (1..4) of the flag-synchronised two-shot paths (default 1)
``TDX_NVLS_BATCH``     NVLS two-shot: rows whose switch-side sums are requested together (1..4, default 1)
``TDX_LOG``            Python logging level of the package logger
``TDX_NVTX``           ``1`` opens an NVTX range around every public op and decoder layer
                       (read by ``utils/tracing.py``)
``TDX_POLICY_JSON``    path of a measured crossover table to load at ``setup_env``
=====================  ============================================================
"""
from __future__ import annotations

import json
import logging
import os
from dataclasses import dataclass, field
from typing import Dict, Tuple

ALGO_CODES = {
    "auto": 0,
    "local": 1,
    "oneshot": 2,
    "twoshot": 3,
    "twoshot_barrier": 4,
    "nvls_oneshot": 5,
    "nvls_twoshot": 6,
    "oneshot_mc": 7,
    "twoshot_mc": 8,
}
ALGO_NAMES = {v: k for k, v in ALGO_CODES.items()}

OUT_SAME, OUT_FP8_TOKEN, OUT_FP8_BLOCK128 = 0, 1, 2


@dataclass
class Config:
    algo: str = "auto"
    timeout_ms: int = 5000
    lamport_mb: int = 72
    nvls: bool = True
    # nranks -> (oneshot_max_bytes, lamport_max_bytes, mc_oneshot, mc_twoshot, nvls_min_bytes), -1 = keep the
    # built-in value; empty = built-in defaults
    policy: Dict[int, Tuple[int, ...]] = field(default_factory=dict)

    @staticmethod
    def from_env() -> "Config":
        c = Config()
        c.algo = os.environ.get("TDX_ALGO", c.algo).lower()
        if c.algo not in ALGO_CODES:
            raise ValueError(f"TDX_ALGO={c.algo!r}: expected one of {sorted(ALGO_CODES)}")
        c.timeout_ms = int(os.environ.get("TDX_TIMEOUT_MS", c.timeout_ms))
        c.lamport_mb = int(os.environ.get("TDX_LAMPORT_MB", c.lamport_mb))
        c.nvls = os.environ.get("TDX_NVLS", "1") not in ("0", "false", "off")
        path = os.environ.get("TDX_POLICY_JSON")
        if path:
            c.load_policy(path)
        level = os.environ.get("TDX_LOG")
        if level:
            logging.getLogger("torch_dist_ext_b200").setLevel(level.upper())
        return c

    def load_policy(self, path: str) -> None:
        """Read ``{"<nranks>": {"oneshot_max_bytes": .., "lamport_max_bytes": .., "mc_oneshot": 0|1,
        "mc_twoshot": 0|1, "nvls_min_bytes": ..}, ...}`` (the last three are optional)."""
        with open(path) as f:
            table = json.load(f)
        for k, v in table.items():
            self.policy[int(k)] = (int(v["oneshot_max_bytes"]), int(v["lamport_max_bytes"]), int(v.get("mc_oneshot", -1)),
                                   int(v.get("mc_twoshot", -1)), int(v.get("nvls_min_bytes", -1)))

    @property
    def algo_code(self) -> int:
        return ALGO_CODES[self.algo]


config = Config.from_env()
