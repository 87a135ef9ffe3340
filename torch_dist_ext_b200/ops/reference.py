"""Pure-PyTorch statement of the fused op: the oracle for every kernel test and the CPU/gloo
path of the library.

Math (identical to the reference's kernels, src/common/all_reduce_fusion_impl.h:280-298,
:316-340, :381-393)::

    s            = T( sum_r float(in_r) )            fp32, rank order, one rounding
    residual_out = T( float(s) + float(residual_in) )
    rstd         = rsqrt( mean_h float(residual_out)^2 + eps )
    y            = float(residual_out) * rstd * float(gamma)
    norm_out     = T(y)                               | e4m3(y / scale)

fp8 (NVIDIA e4m3fn, max 448, saturating): per-token ``scale = max(amax_h |y|, 1e-10) / 448``
with scales of shape ``[tokens, 1]``; 1x128 block scaling uses one such scale per 128
consecutive columns, shape ``[tokens, hidden // 128]``. ``q = e4m3(y * (1 / scale))``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

FP8_MAX = 448.0
AMAX_FLOOR = 1e-10
OUT_SAME, OUT_FP8_TOKEN, OUT_FP8_BLOCK128 = 0, 1, 2


def _to_fp8(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def quantize_fp8(y: torch.Tensor, out_mode: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise fp32 ``y`` [tokens, hidden] -> (e4m3 tensor, fp32 scales)."""
    y = y.float()
    tokens, hidden = y.shape
    if out_mode == OUT_FP8_TOKEN:
        amax = y.abs().amax(dim=-1, keepdim=True).clamp_min(AMAX_FLOOR)
        scale = amax / FP8_MAX
        return _to_fp8(y * (1.0 / scale)), scale
    if out_mode == OUT_FP8_BLOCK128:
        assert hidden % 128 == 0, "1x128 block scaling needs hidden % 128 == 0"
        yb = y.view(tokens, hidden // 128, 128)
        amax = yb.abs().amax(dim=-1, keepdim=True).clamp_min(AMAX_FLOOR)
        scale = amax / FP8_MAX
        return _to_fp8(yb * (1.0 / scale)).view(tokens, hidden), scale.squeeze(-1)
    raise ValueError(f"not an fp8 output mode: {out_mode}")


def dequantize_fp8(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    tokens, hidden = q.shape
    if scale.numel() == tokens:
        return q.float() * scale.view(tokens, 1)
    return (q.float().view(tokens, -1, 128) * scale.view(tokens, -1, 1)).view(tokens, hidden)


def residual_rmsnorm_reference(summed: torch.Tensor, residual: Optional[torch.Tensor], gamma: torch.Tensor,
                               eps: float, out_mode: int = OUT_SAME):
    """Everything after the all-reduce. ``summed`` is fp32 (the exact sum over ranks).

    Returns ``(norm_out, residual_out, scales-or-None)``.
    """
    dtype = gamma.dtype
    s = summed.float().to(dtype)
    res_out = s if residual is None else (s.float() + residual.float()).to(dtype)
    x = res_out.float()
    rstd = torch.rsqrt(x.pow(2).sum(dim=-1, keepdim=True) / x.shape[-1] + eps)
    y = x * rstd * gamma.float()
    if out_mode == OUT_SAME:
        return y.to(dtype), res_out, None
    q, scale = quantize_fp8(y, out_mode)
    return q, res_out, scale


def fused_allreduce_rms_reference(inputs: Sequence[torch.Tensor], residual: Optional[torch.Tensor],
                                  gamma: torch.Tensor, eps: float, out_mode: int = OUT_SAME):
    """Single-process oracle: ``inputs[r]`` is rank r's partial sum."""
    acc = torch.zeros_like(inputs[0], dtype=torch.float32)
    for t in inputs:  # rank order, fp32
        acc = acc + t.float()
    return residual_rmsnorm_reference(acc, residual, gamma, eps, out_mode)


def fused_allreduce_rms_distributed(allreduce_in: torch.Tensor, residual: Optional[torch.Tensor],
                                    gamma: torch.Tensor, eps: float, out_mode: int = OUT_SAME,
                                    group: Optional[dist.ProcessGroup] = None):
    """Multi-process statement of the op over any torch.distributed backend (gloo on CPU).

    The sum is formed in fp32 in rank order (all-gather + ordered add) so that every rank gets
    bit-identical results, as the kernels guarantee.
    """
    world = dist.get_world_size(group)
    parts: List[torch.Tensor] = [torch.empty_like(allreduce_in, dtype=torch.float32) for _ in range(world)]
    dist.all_gather(parts, allreduce_in.float().contiguous(), group=group)
    return fused_allreduce_rms_reference(parts, residual, gamma, eps, out_mode)


def scatter_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows owned by ``rank`` in the round-robin layout of the reduce-scatter variant."""
    return t[rank::world].contiguous()


def greedy_sample_sharded(logits: torch.Tensor, rank: int, world: int, index_base: int,
                          group: Optional["dist.ProcessGroup"] = None) -> torch.Tensor:
    """Arg-max over a vocabulary sharded across ranks, in plain PyTorch: the oracle of ops.sampling."""
    val, idx = logits.float().max(dim=-1)
    idx = idx + index_base
    if world == 1:
        return idx
    packed = torch.stack([val, idx.float()], dim=-1).contiguous()
    parts = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(parts, packed, group=group)
    allp = torch.stack(parts)                                                  # [world, tokens, 2]
    best = allp[..., 0].argmax(dim=0)
    return allp[best, torch.arange(logits.shape[0], device=logits.device), 1].long()


def linear_rope_kv_reference(a: torch.Tensor, w: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor,
                             k_cache: torch.Tensor, v_cache: torch.Tensor, q_heads: int, kv_heads: int) -> torch.Tensor:
    """PyTorch statement of ``ops.gemm.linear_rope_kv`` in fp32: the fused qkv projection ``a @ w^T`` with query and key
    heads rotated (rotate-half, head dimension 128) by the angle of ``positions[t]``; the rotated key row and the value row
    of token ``t`` are written into ``k_cache`` / ``v_cache`` ``[B, S, kv_heads, 128]`` at ``[t, positions[t]]``. Returns
    the rotated ``[T, (q_heads + 2 kv_heads) * 128]`` rows in fp32. (The reference library has no counterpart: its only
    op is the fused all-reduce, src/ops/all_reduce_fusion.cpp:120-173.)"""
    t = a.shape[0]
    qkv = a.float() @ w.float().t()
    q = qkv[:, : q_heads * 128].view(t, q_heads, 128)
    k = qkv[:, q_heads * 128: (q_heads + kv_heads) * 128].view(t, kv_heads, 128)
    v = qkv[:, (q_heads + kv_heads) * 128:].view(t, kv_heads, 128)
    cs = cos_sin_cache[positions].float()
    cos, sin = cs[:, None, :64], cs[:, None, 64:]

    def rotate(x):
        lo, hi = x[..., :64], x[..., 64:]
        return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)

    q, k = rotate(q), rotate(k)
    rows = torch.arange(t, device=a.device)
    k_cache[rows, positions] = k.to(k_cache.dtype)
    v_cache[rows, positions] = v.to(v_cache.dtype)
    return torch.cat([q.reshape(t, -1), k.reshape(t, -1), v.reshape(t, -1)], dim=1)


def linear_silu_mul_reference(a: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """PyTorch statement of ``ops.gemm.linear_silu_mul`` in fp32: ``silu(a @ w_gate^T) * (a @ w_up^T)`` for
    ``w_gate_up [2 ffn, K]`` with the gate rows first."""
    ffn = w_gate_up.shape[0] // 2
    gu = a.float() @ w_gate_up.float().t()
    return torch.nn.functional.silu(gu[:, :ffn]) * gu[:, ffn:]
