"""Python entry points of the fused all-reduce + residual + RMSNorm (+fp8 quant) op.

``allreduce_rms`` has the reference's exact signature and return order
(torch_dist_ext/__init__.py:64-73: ``(norm_out, residual_out)``). The other functions expose
what the reference's README promises but its code does not contain (fp8 quantised output) and
the reduce-scatter variant used by sequence-parallel tensor-parallel layers.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from ..utils.tracing import traced
from ..parallel import comm as _comm
from ..utils.config import ALGO_CODES, OUT_FP8_BLOCK128, OUT_FP8_TOKEN, OUT_SAME, config
from . import reference as _ref


def _algo_code(algo) -> int:
    if algo is None:
        return config.algo_code
    if isinstance(algo, int):
        return algo
    return ALGO_CODES[algo]


def _cpu_path(allreduce_in, residual_in, rms_gamma, eps, out_mode, scatter_only):
    c = _comm.get_comm()
    if c.world_size > 1:
        norm, res, scale = _ref.fused_allreduce_rms_distributed(allreduce_in, residual_in, rms_gamma, eps, out_mode, c.group)
    else:
        norm, res, scale = _ref.fused_allreduce_rms_reference([allreduce_in], residual_in, rms_gamma, eps, out_mode)
    if scatter_only:
        norm, res = norm[c.rank::c.world_size].contiguous(), res[c.rank::c.world_size].contiguous()
        scale = None if scale is None else scale[c.rank::c.world_size].contiguous()
    return norm, res, scale


@traced("tdx.fused_allreduce_rms")
def fused_allreduce_rms(allreduce_in: torch.Tensor, residual_in: Optional[torch.Tensor], rms_gamma: torch.Tensor,
                        eps: float, workspace: Optional[torch.Tensor] = None, *, out_mode: int = OUT_SAME,
                        algo=None, scatter_only: bool = False, want_residual: bool = True,
                        ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """All-reduce ``allreduce_in`` over the registered ranks, add ``residual_in``, RMS-normalise.

    Returns ``(norm_out, residual_out, scales)``; ``scales`` is None unless an fp8 mode is chosen.
    With ``scatter_only`` each rank gets only the rows ``rank::world_size`` (and ``residual_in`` is
    that rank's row shard), i.e. reduce-scatter + residual + RMSNorm.
    """
    if not allreduce_in.is_cuda:
        if scatter_only and residual_in is not None:
            raise NotImplementedError("scatter_only with a sharded residual is CUDA-only")
        return _cpu_path(allreduce_in, residual_in, rms_gamma, eps, out_mode, scatter_only)
    if allreduce_in.dtype == torch.float64:
        # The reference instantiates its kernels for double through its dispatch macro
        # (src/ops/all_reduce_fusion.cpp:29-33) but still accumulates, adds and normalises in fp32
        # (src/common/all_reduce_fusion_impl.h:280-298, :316-340), so its float64 results are fp32 values stored
        # as doubles. The same values come out of the fp32 kernels around two conversions.
        norm, res, scales = fused_allreduce_rms(
            allreduce_in.float(), None if residual_in is None else residual_in.float(), rms_gamma.float(), eps, workspace,
            out_mode=out_mode, algo=algo, scatter_only=scatter_only, want_residual=want_residual)
        return (norm.double() if out_mode == OUT_SAME else norm), (None if res is None else res.double()), scales
    c = _comm.get_comm()
    if workspace is None:
        workspace = c.get_workspace(allreduce_in)
    hidden = allreduce_in.shape[-1]
    tokens = allreduce_in.numel() // hidden
    n = c.world_size
    rows = (tokens + n - 1) // n if scatter_only else tokens
    lead = allreduce_in.shape[:-1] if not scatter_only else (rows,)
    residual_out = allreduce_in.new_empty(*lead, hidden) if want_residual else None
    if out_mode == OUT_SAME:
        norm_out = allreduce_in.new_empty(*lead, hidden)
        scales = None
    else:
        norm_out = torch.empty(*lead, hidden, dtype=torch.float8_e4m3fn, device=allreduce_in.device)
        ncol = 1 if out_mode == OUT_FP8_TOKEN else hidden // 128
        scales = torch.empty(rows, ncol, dtype=torch.float32, device=allreduce_in.device)
    used = _lib.ops().allreduce_rms_fusion_ex(allreduce_in, residual_in, rms_gamma, residual_out, norm_out, scales,
                                              eps, workspace, out_mode, _algo_code(algo), scatter_only)
    c.algo_counts[used] = c.algo_counts.get(used, 0) + 1
    return norm_out, residual_out, scales


@traced("tdx.allreduce_rms_pinned")
def allreduce_rms_pinned(allreduce_in: torch.Tensor, residual_in: Optional[torch.Tensor], rms_gamma: torch.Tensor,
                         eps: float, *, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, algo=None,
                         ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The fused op for data that starts and ends in pinned host memory.

    ``allreduce_in`` / ``residual_in`` may be pinned CPU tensors (or device tensors), ``out`` is an
    optional pair of pinned ``(norm_out, residual_out)`` tensors to fill (allocated when omitted;
    reuse them across calls). The kernel reads its inputs and writes its outputs over PCIe itself:
    no staging copies, one launch, and with the two-shot algorithms each rank fetches only the
    residual rows it owns. ``rms_gamma`` stays on the device (every row re-reads it). The outputs
    are valid once the launching stream has been synchronised. Returns ``(norm_out, residual_out)``.
    """
    c = _comm.get_comm()
    if c.comm is None:
        raise RuntimeError("allreduce_rms_pinned needs the CUDA workspace (setup_env on a machine with a GPU)")
    if out is None:
        out = (torch.empty(allreduce_in.shape, dtype=allreduce_in.dtype).pin_memory(),
               torch.empty(allreduce_in.shape, dtype=allreduce_in.dtype).pin_memory())
    norm_out, residual_out = out
    workspace = c.get_workspace(rms_gamma)
    used = _lib.ops().allreduce_rms_fusion_hostio(allreduce_in, residual_in, rms_gamma, residual_out, norm_out, None,
                                                  eps, workspace, OUT_SAME, _algo_code(algo), False)
    c.algo_counts[used] = c.algo_counts.get(used, 0) + 1
    return norm_out, residual_out


def allreduce_rms_fp8(allreduce_in, residual_in, rms_gamma, eps, workspace=None, *, block_scaled: bool = False,
                      algo=None):
    """Fused op with e4m3 output. Returns ``(norm_fp8, scales, residual_out)``."""
    mode = OUT_FP8_BLOCK128 if block_scaled else OUT_FP8_TOKEN
    norm, res, scales = fused_allreduce_rms(allreduce_in, residual_in, rms_gamma, eps, workspace, out_mode=mode, algo=algo)
    return norm, scales, res


def reduce_scatter_rms(allreduce_in, residual_shard, rms_gamma, eps, workspace=None, *, out_mode: int = OUT_SAME,
                       algo=None):
    """Reduce-scatter + residual + RMSNorm on this rank's rows (``rank::world_size``)."""
    return fused_allreduce_rms(allreduce_in, residual_shard, rms_gamma, eps, workspace, out_mode=out_mode,
                               algo=algo, scatter_only=True)
