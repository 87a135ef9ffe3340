"""GEMMs fused with their collectives (one kernel each, data moved by peer loads/stores).

``gemm_allreduce_rms``  row-parallel linear + all-reduce (or reduce-scatter) + residual + RMSNorm:
                        the o_proj / down_proj step of a tensor-parallel decoder layer.
``allgather_gemm``      all-gather of sequence-parallel rows + column-parallel linear:
                        the qkv / gate-up step that follows a reduce-scattered norm.

``allgather_gemm`` and the e4m3 form of ``gemm_allreduce_rms`` are decode-sized paths (one CTA per tile, all CTAs
resident at once); for more tokens they fall back to the tcgen05 GEMM followed / preceded by the fused all-reduce
op. With bf16 operands ``gemm_allreduce_rms`` stays fused at any token count that fits the Lamport buffers: a
persistent kernel (one CTA per SM) walks the tiles.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from ..utils.tracing import traced
from ..parallel import comm as _comm
from ..utils.config import OUT_FP8_BLOCK128, OUT_SAME
from . import gemm as _gemm
from .fused_allreduce import fused_allreduce_rms

_SM_COUNT = 148


def _oneshot_limit(world: int) -> int:
    """Message bytes up to which the all-reduce op takes its one-shot route at this rank count (the measured table)."""
    try:
        return int(_lib.ops().get_policy(world)[0])
    except Exception:
        return 512 << 10


def _fits(tokens: int, rows: int) -> bool:
    bn = 16 if tokens <= 16 else 64
    return ((rows + 127) // 128) * ((tokens + bn - 1) // bn) <= _SM_COUNT


@traced("tdx.gemm_allreduce_rms")
def gemm_allreduce_rms(a: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor], gamma: torch.Tensor,
                       eps: float, *, out_mode: int = OUT_SAME, scatter_only: bool = False,
                       want_residual: bool = True, force_unfused: bool = False, splits: int = 0,
                       a_scale: Optional[torch.Tensor] = None, w_scale: Optional[torch.Tensor] = None,
                       one_hop: Optional[bool] = None,
                       ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``y = all_reduce(a @ w.T); res = y + residual; norm = rmsnorm(res) * gamma``.

    ``a [tokens, K_shard]``, ``w [hidden, K_shard]``: bf16, or e4m3 with ``a_scale [tokens, K/128]`` (one scale per
    token and 128-wide K block) and ``w_scale [hidden/128, K/128]`` (one per 128 x 128 block), fp32. Residual, gamma
    and the non-quantised outputs are bf16. Returns ``(norm, res, scales)``; with ``scatter_only`` only the rows
    ``rank::world`` (and ``residual`` is that row shard).

    ``one_hop``: the tail of the fused kernel. True: every finished tile is pushed into EVERY rank's buffer (one
    ``multimem.st`` per vector where NVSwitch multicast is mapped) and each rank reduces all rows itself - one trip
    through NVSwitch, the choice for decode sizes; False: reduce-scatter to the rows' owners, reduce once, gather
    back - two trips, N times fewer bytes to reduce. None: one hop up to the message size at which the all-reduce
    op leaves its one-shot algorithm (the same measured limit), replicated output only.
    """
    c = _comm.get_comm()
    tokens, hidden = a.shape[0], w.shape[0]
    fp8 = a.dtype == torch.float8_e4m3fn
    if fp8 and w.shape[0] != gamma.shape[0]:
        hidden = gamma.shape[0]         # weights padded to a multiple of 128 rows
    n = c.world_size
    if not _fits(tokens, hidden):
        # beyond one CTA per tile: the persistent kernel, bf16 operands, gather slots + result rows in one Lamport buffer
        groups = (tokens + n - 1) // n
        need = n * groups * hidden * 2 + (0 if scatter_only else tokens * (hidden * 2 + 16))
        fused = not fp8 and a.dtype == torch.bfloat16 and need <= c.lamport_bytes
    else:
        fused = True
    if force_unfused or not fused or hidden % 128 or out_mode not in (OUT_SAME, OUT_FP8_BLOCK128):
        if fp8:
            y = _gemm.linear_fp8_blockscaled(a, a_scale, w, w_scale)
            y = y[:, :hidden] if y.shape[1] != hidden else y
        else:
            y = _gemm.linear(a, w)
        return fused_allreduce_rms(y, residual, gamma, eps, out_mode=out_mode, scatter_only=scatter_only,
                                   want_residual=want_residual)
    rows = (tokens + n - 1) // n if scatter_only else tokens
    act_dtype = torch.bfloat16 if fp8 else a.dtype
    res_out = torch.empty(rows, hidden, dtype=act_dtype, device=a.device) if want_residual else None
    if out_mode == OUT_SAME:
        norm, scales = torch.empty(rows, hidden, dtype=act_dtype, device=a.device), None
    else:
        norm = torch.empty(rows, hidden, dtype=torch.float8_e4m3fn, device=a.device)
        scales = torch.empty(rows, hidden // 128, dtype=torch.float32, device=a.device)
    ws, counters, status = _gemm._workspace(a.device)
    if one_hop is None:
        one_hop = (not scatter_only) and _fits(tokens, hidden) and tokens * hidden * 2 <= _oneshot_limit(n)
    one_hop = bool(one_hop) and not scatter_only and _fits(tokens, hidden) and n * tokens * hidden * 2 <= c.lamport_bytes
    _lib.ops().gemm_ar_rmsnorm(a, w[:hidden] if w.shape[0] != hidden else w, residual, gamma, res_out, norm, scales, eps,
                               c.get_workspace(a), out_mode, scatter_only, status, splits, ws, counters,
                               a_scale.contiguous() if fp8 else None, w_scale.contiguous() if fp8 else None, one_hop)
    return norm, res_out, scales


@traced("tdx.allgather_gemm")
def allgather_gemm(x_shard: torch.Tensor, w: torch.Tensor, tokens: int, *, force_unfused: bool = False) -> torch.Tensor:
    """``gather(x_shard) @ w.T`` where rank r holds the rows ``r::world`` of the ``[tokens, K]`` input."""
    c = _comm.get_comm()
    n = c.world_size
    if force_unfused or not _fits(tokens, w.shape[0]) or tokens * w.shape[1] * 2 > (32 << 20):
        import torch.distributed as dist

        rows = (tokens + n - 1) // n
        pad = torch.zeros(rows, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
        pad[: x_shard.shape[0]] = x_shard
        parts = [torch.empty_like(pad) for _ in range(n)]
        if n > 1:
            dist.all_gather(parts, pad, group=c.group)
        else:
            parts = [pad]
        full = torch.stack(parts, dim=1).reshape(rows * n, -1)[:tokens].contiguous()
        return _gemm.linear(full, w)
    out = torch.empty(tokens, w.shape[0], dtype=x_shard.dtype, device=x_shard.device)
    status = _gemm._workspace(x_shard.device)[2]
    _lib.ops().ag_gemm(x_shard.contiguous(), w, out, tokens, c.get_workspace(x_shard), status)
    return out
