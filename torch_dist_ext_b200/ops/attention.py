"""Attention for grouped-query heads of dimension 128: decode (one new token per sequence over a
contiguous bf16 KV cache; tcgen05 kernel, or the SIMT kernel with ``TDX_ATTN_TC=0``) and causal attention over one
prompt (tcgen05 kernel)."""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .. import _lib
from ..utils.tracing import traced

_scratch = {}
_TC_DEFAULT = os.environ.get("TDX_ATTN_TC", "1") not in ("0", "", "false", "off")


def _partial(device, floats: int) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _scratch or _scratch[key].numel() < floats:
        # zeroed: the first 4096 words are arrival counters that the kernel expects (and leaves) at zero
        _scratch[key] = torch.zeros(max(floats, 1 << 20), dtype=torch.float32, device=device)
    return _scratch[key]


# Measured on a B200 for the tensor-core kernel (2048 positions, 1 to 64 sequences, 1 and 8 KV heads): a CTA takes
# about 1.0 us per 128-position chunk while the grid is small and 13.1 ns x (CTAs in flight) once the grid saturates
# HBM; an unsplit launch costs about 2.6 us besides, a split one 9 us plus 0.4 us per split (partial results through
# L2, the arrival counter and the merge by the last CTA of each group).
_CHUNK_US, _CHUNK_US_PER_CTA, _UNSPLIT_US, _SPLIT_US, _PER_SPLIT_US = 1.0, 0.0131, 2.6, 9.0, 0.4


def _split_cost_us(pairs: int, chunks: int, nsplit: int) -> float:
    ctas = pairs * nsplit
    per_chunk = max(_CHUNK_US, _CHUNK_US_PER_CTA * ctas)
    return -(-chunks // nsplit) * per_chunk + (_UNSPLIT_US if nsplit == 1 else _SPLIT_US + _PER_SPLIT_US * nsplit)


def pick_splits(batch: int, kv_heads: int, max_len: int, sms: int = 148, ctas_per_sm: int = 2) -> int:
    """KV splits of at least 128 positions each, such that the grid fits ONE wave of the CTAs that the SMs hold at a
    time (two per SM for the SIMT kernel, one for the tensor-core kernel; a second, partly filled wave costs more than
    shorter splits save).

    The SIMT kernel takes the most splits that fit. The tensor-core kernel (``ctas_per_sm=1``) takes the split count
    with the least estimated time: a split that leaves some CTAs one chunk more than others (16 chunks over 9 splits)
    is no faster than the next count that divides evenly (8), and once the unsplit grid already covers a third of
    the SMs (64 sequences on one KV head) the merge costs more than the shorter loops save."""
    pairs = batch * kv_heads
    chunks = max(1, (max_len + 127) // 128)
    most = max(1, min((ctas_per_sm * sms) // pairs, chunks))
    if ctas_per_sm != 1:
        return most
    return min(range(1, most + 1), key=lambda n: (_split_cost_us(pairs, chunks, n), n))


@traced("tdx.decode_attention")
def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_lens: torch.Tensor,
                     max_len: int, out: Optional[torch.Tensor] = None, nsplit: Optional[int] = None,
                     tensor_cores: Optional[bool] = None) -> torch.Tensor:
    """``q [B, Hq, 128]``, caches ``[B, S_max, Hkv, 128]``, ``seq_lens`` int32 ``[B]`` -> ``[B, Hq, 128]``.

    ``max_len`` (a host integer >= every sequence length) only sizes the KV split. ``tensor_cores=True``
    runs both products of every 128-position chunk as tcgen05 MMAs (default: ``TDX_ATTN_TC``, on)."""
    b, hq, d = q.shape
    hkv = k_cache.shape[2]
    use_tc = _TC_DEFAULT if tensor_cores is None else tensor_cores
    if nsplit is None:
        nsplit = pick_splits(b, hkv, max_len, ctas_per_sm=1 if use_tc else 2)
    out = torch.empty(b, hq, d, dtype=q.dtype, device=q.device) if out is None else out
    part = _partial(q.device, 4096 + b * hq * nsplit * (d + 2))
    from . import gemm as _gemm

    op = _lib.ops().attention_decode_tc if use_tc else _lib.ops().attention_decode
    op(q, k_cache, v_cache, seq_lens, out, part, nsplit, 1.0 / math.sqrt(d), _gemm._workspace(q.device)[2])
    return out


@traced("tdx.prefill_attention")
def prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal self-attention over one prompt on the tensor cores: ``q [S, Hq, 128]``, ``k``/``v`` ``[S, Hkv, 128]``
    (views into a fused qkv projection are fine) -> ``[S, Hq, 128]``; query i attends to keys 0..i."""
    s, hq, d = q.shape
    out = torch.empty(s, hq, d, dtype=q.dtype, device=q.device) if out is None else out
    from . import gemm as _gemm

    _lib.ops().attention_prefill_tc(q, k, v, out, 1.0 / math.sqrt(d), _gemm._workspace(q.device)[2])
    return out


def prefill_attention_reference(q, k, v):
    hq, hkv = q.shape[1], k.shape[1]
    kk = k.float().repeat_interleave(hq // hkv, dim=1)
    vv = v.float().repeat_interleave(hq // hkv, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) / math.sqrt(q.shape[-1])
    s = s.masked_fill(torch.ones(q.shape[0], q.shape[0], dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, dim=-1), vv).to(q.dtype)


def decode_attention_reference(q, k_cache, v_cache, seq_lens):
    b, hq, d = q.shape
    hkv = k_cache.shape[2]
    g = hq // hkv
    outs = []
    for i in range(b):
        n = int(seq_lens[i])
        k = k_cache[i, :n].float().repeat_interleave(g, dim=1)   # [n, hq, d]
        v = v_cache[i, :n].float().repeat_interleave(g, dim=1)
        s = torch.einsum("hd,nhd->hn", q[i].float(), k) / math.sqrt(d)
        outs.append(torch.einsum("hn,nhd->hd", torch.softmax(s, dim=-1), v))
    return torch.stack(outs).to(q.dtype)
