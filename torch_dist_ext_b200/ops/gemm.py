"""Linear layers on the 5th-generation tensor cores (tcgen05 / TMEM), bf16 / fp16 / fp8.

``linear(a, w)`` computes ``a @ w.T`` for ``a [M, K]`` and ``w [N, K]`` (the ``nn.Linear`` weight
layout). Small ``M`` (decode) runs "swapped": the weight rows fill the 128-row side of the MMA
tile and the tokens its narrow side, so a decode step streams the weights once at full tile
efficiency; K is split over CTAs until the grid covers the 148 SMs.

``linear_fp8_blockscaled`` multiplies e4m3 activations with 1x128 scales by e4m3 weights with
128x128 scales (fp32 scales), promoting every 128-wide K block in fp32.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from .. import _lib
from ..utils.tracing import traced

_SM_COUNT = 148
_ws = {}


_PAIR_DEFAULT = os.environ.get("TDX_GEMM_PAIR", "1") not in ("0", "", "false", "off")
_PERSIST_DEFAULT = os.environ.get("TDX_GEMM_PERSIST", "1") not in ("0", "", "false", "off")


def _workspace(device: torch.device):
    """Per-device split-K scratch: zeroed once; every kernel leaves it zeroed again."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _ws:
        _ws[key] = (torch.zeros(8 << 20, dtype=torch.float32, device=device),      # 32 MiB
                    torch.zeros(4096, dtype=torch.int32, device=device),
                    torch.zeros(1, dtype=torch.int32, device=device))
    return _ws[key]


_pair_ws = {}


def _pair_scratch(device: torch.device) -> torch.Tensor:
    """Scratch of the CTA-pair kernel's tail split: fp32 partial tiles, contents undefined between calls (unlike the
    split-K scratch above, which every kernel leaves zeroed)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _pair_ws:
        _pair_ws[key] = torch.empty(20 << 20, dtype=torch.float32, device=device)      # 80 MiB: 73 tiles x 4 pieces
    return _pair_ws[key]


def pipeline_status(device=None) -> int:
    """Non-zero if a GEMM pipeline wait ever ran out on this device (reads the device word)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(_workspace(dev)[2].item())


def _pick_bn(rows: int, cap: int) -> int:
    for bn in (16, 32, 64, 128, 256):
        if bn <= cap and rows <= bn:
            return bn
    return cap


def plan(m: int, n: int, k: int, elem_size: int = 2, scaled: bool = False) -> Tuple[bool, int, int]:
    """(swap, block_n, splits) for ``[m, k] x [n, k]^T``."""
    cap = 64 if scaled else 256
    swap = m <= 128 if not scaled else True
    x_rows, y_rows = (n, m) if swap else (m, n)
    bn = _pick_bn(y_rows, cap)
    if not swap and n >= 256:
        bn = 256 if (m // 128) * (n // 256) >= _SM_COUNT else 128
    tiles = ((x_rows + 127) // 128) * ((y_rows + bn - 1) // bn)
    kblocks = k // (128 // elem_size)
    splits = 1
    if tiles < _SM_COUNT:
        splits = max(1, min(kblocks // 2 if kblocks >= 2 else 1, _SM_COUNT // tiles))
    return swap, bn, splits


@traced("tdx.linear")
def linear(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, *, out_dtype=None,
           swap: Optional[bool] = None, block_n: int = 0, splits: Optional[int] = None,
           cta_pair: Optional[bool] = None, persistent: Optional[bool] = None) -> torch.Tensor:
    """``a [M, K] @ w [N, K]^T -> [M, N]`` (bf16 / fp16 / e4m3 operands, fp32 accumulation).

    ``cta_pair=True`` runs prefill-sized problems (M, N >= 256) on 256 x 256 tiles computed by pairs of
    CTAs (``tcgen05.mma.cta_group::2``) that walk the tiles persistently with the accumulator double-buffered in
    tensor memory; the default follows ``TDX_GEMM_PAIR`` (on: it is the fastest kernel for these shapes). ``persistent=True`` runs
    them on a persistent grid (one CTA per SM, accumulator double-buffered in tensor memory so that the epilogue
    of a tile overlaps the main loop of the next); the default follows ``TDX_GEMM_PERSIST`` (on)."""
    assert a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "linear: a [M, K], w [N, K]"
    m, k = a.shape
    n = w.shape[0]
    # an explicit choice of one kernel is not overridden by the default of the other
    use_pair = cta_pair if cta_pair is not None else (_PAIR_DEFAULT and persistent is None)
    use_persistent = persistent if persistent is not None else (_PERSIST_DEFAULT and not use_pair)
    if use_pair and m >= 256 and n >= 256 and not swap and splits in (None, 1):
        if out is None:
            dt = out_dtype or (torch.bfloat16 if a.element_size() == 1 else a.dtype)
            out = torch.empty(m, n, dtype=dt, device=a.device)
        _, counters, status = _workspace(a.device)
        _lib.ops().gemm_tn_pair(a, w, out, n, 1, status, _pair_scratch(a.device), counters)   # K-split of a partly filled last round
        return out
    if (use_persistent or (use_pair and persistent is None and _PERSIST_DEFAULT)) and m > 128 and n >= 256 and not swap \
            and splits in (None, 1):
        if out is None:
            dt = out_dtype or (torch.bfloat16 if a.element_size() == 1 else a.dtype)
            out = torch.empty(m, n, dtype=dt, device=a.device)
        _lib.ops().gemm_tn_persistent(a, w, out, n, 1, _workspace(a.device)[2])
        return out
    p_swap, p_bn, p_splits = plan(m, n, k, a.element_size())
    swap = p_swap if swap is None else swap
    if block_n == 0:
        block_n = p_bn if swap == p_swap else _pick_bn(m if swap else n, 256)
    splits = p_splits if splits is None else splits
    if out is None:
        dt = out_dtype or (torch.bfloat16 if a.element_size() == 1 else a.dtype)
        out = torch.empty(m, n, dtype=dt, device=a.device)
    ws, counters, status = _workspace(a.device)
    if swap:
        # swapped: X is the weight, which no kernel writes, so its first tiles may be fetched ahead of the stream order
        _lib.ops().gemm_tn(w, a, out, 1, n, block_n, splits, ws, counters, status, None, None, False, False, True)
    else:
        _lib.ops().gemm_tn(a, w, out, n, 1, block_n, splits, ws, counters, status, None, None, False, False)
    return out


@traced("tdx.linear_fp8_blockscaled")
def linear_fp8_blockscaled(a_q: torch.Tensor, a_scale: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor,
                           out: Optional[torch.Tensor] = None, *, out_dtype=torch.bfloat16,
                           splits: Optional[int] = None) -> torch.Tensor:
    """``(a_q * a_scale) @ (w_q * w_scale)^T`` with ``a_scale [M, K/128]`` and ``w_scale [N/128, K/128]``."""
    m, k = a_q.shape
    n = w_q.shape[0]
    _, bn, p_splits = plan(m, n, k, 1, scaled=True)
    splits = p_splits if splits is None else splits
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a_q.device)
    ws, counters, status = _workspace(a_q.device)
    _lib.ops().gemm_tn(w_q, a_q, out, 1, n, bn, splits, ws, counters, status, w_scale.contiguous(),
                       a_scale.contiguous(), False, True, True)
    return out


def fused_epilogue_fits(tokens: int, k: int, elem_size: int = 2, scaled: bool = False) -> bool:
    """Whether ``linear_rope_kv`` / ``linear_silu_mul`` can take the problem: the weights must sit on the 128-row side of
    the tile (decode-sized token counts; always for block-scaled operands) and K must span at least two 128-byte blocks
    (the fused epilogues live in the split-K finalizer)."""
    return plan(tokens, 256, k, elem_size, scaled)[0] and k // (128 // elem_size) >= 2


@traced("tdx.linear_rope_kv")
def linear_rope_kv(a: torch.Tensor, w: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, q_heads: int, kv_heads: int, *,
                   a_scale: Optional[torch.Tensor] = None, w_scale: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fused qkv projection of a decode step with the rotary embedding and the KV append in the GEMM's own epilogue:
    ``qkv = a [T, K] @ w [(q_heads + 2 kv_heads) * 128, K]^T``, query and key heads rotated (rotate-half) by the angle of
    ``positions[t]``, the rotated key row and the value row of token ``t`` written to ``k_cache`` / ``v_cache``
    ``[B, S, kv_heads, 128]`` at ``[t, positions[t]]``. Returns the rotated ``[T, (q_heads + 2 kv_heads) * 128]`` bf16 rows.
    One kernel where ``linear`` + ``rope_append_kv_`` are two. e4m3 operands take ``a_scale [T, K/128]`` and
    ``w_scale [N/128, K/128]``. PyTorch statement: ``ops.reference.linear_rope_kv_reference``."""
    m, k = a.shape
    n = w.shape[0]
    scaled = w_scale is not None
    assert n == (q_heads + 2 * kv_heads) * 128, "linear_rope_kv: w must hold (q_heads + 2 kv_heads) heads of 128 rows"
    assert fused_epilogue_fits(m, k, a.element_size(), scaled), "linear_rope_kv: decode-sized token counts only"
    _, bn, splits = plan(m, n, k, a.element_size(), scaled)
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16 if a.element_size() == 1 else a.dtype, device=a.device)
    ws, counters, status = _workspace(a.device)
    _lib.ops().gemm_tn_rope_kv(w, a, out, bn, max(2, splits), ws, counters, status,
                               w_scale.contiguous() if scaled else None, a_scale.contiguous() if scaled else None,
                               positions, cos_sin_cache, k_cache, v_cache, q_heads, kv_heads)
    return out


@traced("tdx.linear_silu_mul")
def linear_silu_mul(a: torch.Tensor, w_gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(a @ w_gate^T) * (a @ w_up^T)`` for ``w_gate_up [2 ffn, K]`` (gate rows, then up rows; bf16 / fp16; ffn a
    multiple of 64) in ONE kernel: every tile of the GEMM is loaded as 64 gate rows plus the 64 up rows of the same
    features, and the split-K finalizer applies the activation. Decode-sized token counts. PyTorch statement:
    ``ops.reference.linear_silu_mul_reference``."""
    m, k = a.shape
    ffn = w_gate_up.shape[0] // 2
    assert w_gate_up.shape[0] == 2 * ffn and ffn % 64 == 0, "linear_silu_mul: w must be [2 ffn, K] with ffn a multiple of 64"
    assert a.element_size() == 2 and fused_epilogue_fits(m, k), "linear_silu_mul: 16-bit operands, decode-sized token counts"
    _, bn, splits = plan(m, 2 * ffn, k, 2)
    if out is None:
        out = torch.empty(m, ffn, dtype=a.dtype, device=a.device)
    ws, counters, status = _workspace(a.device)
    _lib.ops().gemm_tn_silu_mul(w_gate_up, a, out, bn, max(2, splits), ws, counters, status)
    return out


def quantize_weight_block128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """e4m3 weights with one fp32 scale per 128x128 block (PyTorch; done once at load time)."""
    n, k = w.shape
    assert n % 128 == 0 and k % 128 == 0
    blocks = w.float().view(n // 128, 128, k // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3), keepdim=True).clamp_min(1e-10)
    scale = amax / 448.0
    q = (blocks / scale).clamp(-448, 448).to(torch.float8_e4m3fn).view(n, k)
    return q, scale.view(n // 128, k // 128).contiguous()
