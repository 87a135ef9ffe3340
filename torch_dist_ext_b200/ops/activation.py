"""SiLU(gate) * up for gated MLPs, optionally quantising the result for an fp8 down projection."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from ..utils.tracing import traced


@traced("tdx.silu_mul")
def silu_mul(gate_up: torch.Tensor, quant_block128: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``gate_up`` is ``[..., 2 * inter]`` with the gate in the first half. Returns ``(out, scales)``."""
    inter = gate_up.shape[-1] // 2
    rows = gate_up.numel() // gate_up.shape[-1]
    shape = gate_up.shape[:-1] + (inter,)
    if quant_block128:
        out = torch.empty(shape, dtype=torch.float8_e4m3fn, device=gate_up.device)
        scales = torch.empty(rows, inter // 128, dtype=torch.float32, device=gate_up.device)
    else:
        out, scales = torch.empty(shape, dtype=gate_up.dtype, device=gate_up.device), None
    _lib.ops().silu_mul(gate_up, out, scales)
    return out, scales
