"""fp8 e4m3 quantisation with dynamic scales (per token, or per 1x128 block)."""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _lib
from ..utils.tracing import traced


@traced("tdx.quant_fp8")
def quant_fp8(x: torch.Tensor, block_scaled: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(q, scales)`` with ``x ~= q.float() * scales`` (scales ``[rows, 1]`` or ``[rows, cols/128]``)."""
    cols = x.shape[-1]
    rows = x.numel() // cols
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.empty(rows, cols // 128 if block_scaled else 1, dtype=torch.float32, device=x.device)
    _lib.ops().quant_fp8(x.contiguous(), q, scales, block_scaled)
    return q, scales
