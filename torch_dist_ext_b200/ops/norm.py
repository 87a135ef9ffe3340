"""RMSNorm family without communication: (residual add +) RMSNorm (+ fp8 quantisation).

This is the single-rank form of the fused op - the same kernel body that the all-reduce paths
use for their epilogue - and the "separate kernel" of the NCCL baseline.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from ..utils.tracing import traced
from ..utils.config import OUT_FP8_TOKEN, OUT_SAME


@traced("tdx.fused_add_rmsnorm")
def fused_add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], gamma: torch.Tensor, eps: float,
                      out_mode: int = OUT_SAME, want_residual: bool = True,
                      ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``res = x + residual; norm = rmsnorm(res) * gamma``. Returns ``(norm, res, scales)``."""
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    res_out = torch.empty_like(x) if (want_residual and residual is not None) else None
    if out_mode == OUT_SAME:
        norm, scales = torch.empty_like(x), None
    else:
        norm = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        scales = torch.empty(rows, 1 if out_mode == OUT_FP8_TOKEN else hidden // 128, dtype=torch.float32, device=x.device)
    _lib.ops().fused_add_rmsnorm(x, residual, gamma, res_out, norm, scales, eps, out_mode)
    return norm, (res_out if residual is not None else x), scales


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return fused_add_rmsnorm(x, None, gamma, eps, want_residual=False)[0]
