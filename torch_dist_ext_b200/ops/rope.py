"""Rotary position embedding (rotate-half layout, as in Llama), applied in place."""
from __future__ import annotations

import torch

from .. import _lib
from ..utils.tracing import traced


def build_cos_sin_cache(max_pos: int, dim: int, theta: float = 5e5, device="cuda") -> torch.Tensor:
    """fp32 ``[max_pos, dim]`` = ``{cos(pos * inv_freq) | sin(pos * inv_freq)}``."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1).float().to(device).contiguous()


@traced("tdx.rope_")
def rope_(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor) -> None:
    """Rotate ``q`` ``[tokens, q_heads, dim]`` and ``k`` ``[tokens, k_heads, dim]`` in place."""
    _lib.ops().rope_(q, k, positions, cos_sin_cache)


@traced("tdx.rope_append_kv_")
def rope_append_kv_(q, k, v, positions, cos_sin_cache, k_cache, v_cache) -> None:
    """Decode step: rotate ``q``/``k`` in place and append the rotated key row and the value row of
    token ``t`` to ``k_cache``/``v_cache`` ``[B, S, k_heads, dim]`` at ``[t, positions[t]]`` - one kernel."""
    _lib.ops().rope_append_kv_(q, k, v, positions, cos_sin_cache, k_cache, v_cache)


def rope_reference(x: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    cs = cos_sin_cache[positions].float()
    cos, sin = cs[:, None, :half], cs[:, None, half:]
    a, b = x.float()[..., :half], x.float()[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)
