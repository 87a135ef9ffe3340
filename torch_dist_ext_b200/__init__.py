"""torch_dist_ext_b200 - Blackwell-native fused-collective ops for PyTorch.

Public surface (same names, arguments and return layout as the reference package,
torch_dist_ext/__init__.py:41-84)::

    setup_env(rank, world_size, max_size_in_bytes=128 MiB, group=None)
    get_workspace(ref) -> uint8 device tensor (the device-resident peer table)
    allreduce_rms(rank, nranks, allreduce_in, residual_in, rms_gamma, eps, workspace)
        -> (norm_out, residual_out)

plus fp8-quantised and reduce-scatter variants, standalone hot ops, tcgen05 GEMMs fused with
their collectives and Llama-shaped tensor-parallel models (see the sub-packages).
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib
from .ops import reference
from .ops.fused_allreduce import allreduce_rms_fp8, allreduce_rms_pinned, fused_allreduce_rms, reduce_scatter_rms
from .parallel import comm as _comm
from .parallel.comm import CommProcess, get_comm, local_workspaces, setup_env, teardown_env
from .utils.config import ALGO_CODES, OUT_FP8_BLOCK128, OUT_FP8_TOKEN, OUT_SAME, Config, config

__version__ = "0.1.0"

_lib.load()
CommWorkspace = torch.classes.torch_dist_ext.CommWorkspace
allreduce_rms_fusion_impl = torch.ops.torch_dist_ext.allreduce_rms_fusion


@torch.library.custom_op("torch_dist_ext::get_workspace", mutates_args=[])
def get_workspace(ref: torch.Tensor) -> torch.Tensor:
    # An op's output must be a fresh tensor, never a view of memory the library owns, so this returns a
    # copy of the device-resident table and tells the workspace about it (the ops find their workspace by
    # the table's address). The table never changes after registration; the copy holds the same pointers.
    return _comm.get_comm().get_workspace_copy(ref)


@torch.library.register_fake("torch_dist_ext::get_workspace")
def _get_workspace_fake(ref: torch.Tensor) -> torch.Tensor:
    assert _comm.world_size() is not None, "call setup_env first"
    return torch.empty(_comm.table_nbytes(), dtype=torch.uint8, device=ref.device)


def _allreduce_rms_impl(rank: int, nranks: int, allreduce_in: torch.Tensor, residual_in: torch.Tensor,
                        rms_gamma: torch.Tensor, eps: float, workspace: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    c = _comm.get_comm()
    if rank != c.rank or nranks != c.world_size:
        raise ValueError(f"allreduce_rms(rank={rank}, nranks={nranks}) does not match setup_env"
                         f"(rank={c.rank}, world_size={c.world_size})")
    norm_out, residual_out, _ = fused_allreduce_rms(allreduce_in, residual_in, rms_gamma, eps,
                                                    workspace if allreduce_in.is_cuda else None)
    return norm_out, residual_out


# The registered op (with its fake implementation below) is what tracing and export see.
_allreduce_rms_op = torch.library.custom_op("torch_dist_ext::allreduce_rms", _allreduce_rms_impl, mutates_args=[])


def allreduce_rms(rank: int, nranks: int, allreduce_in: torch.Tensor, residual_in: torch.Tensor,
                  rms_gamma: torch.Tensor, eps: float, workspace: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-reduce + residual add + RMSNorm; returns ``(norm_out, residual_out)`` (the reference's
    signature and order, torch_dist_ext/__init__.py:64-73). Plain tensors in eager mode go straight
    to the kernel launch; traced calls and tensor subclasses (fake tensors) go through the
    registered op ``torch_dist_ext::allreduce_rms``, whose Python dispatch costs several times the
    launch itself."""
    if type(allreduce_in) is torch.Tensor and not torch.compiler.is_compiling():
        return _allreduce_rms_impl(rank, nranks, allreduce_in, residual_in, rms_gamma, eps, workspace)
    return _allreduce_rms_op(rank, nranks, allreduce_in, residual_in, rms_gamma, eps, workspace)


@torch.library.register_fake("torch_dist_ext::allreduce_rms")
def _allreduce_rms_fake(rank: int, nranks: int, allreduce_in: torch.Tensor, residual_in: torch.Tensor,
                        rms_gamma: torch.Tensor, eps: float, workspace: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return torch.empty_like(allreduce_in), torch.empty_like(residual_in)


def stats() -> dict:
    """Workspace sizes, epochs, error record and how often each algorithm was chosen."""
    return get_comm().stats()


def check_status() -> None:
    """Raise if any device-side wait timed out since the last reset."""
    get_comm().check()


__all__ = [
    "setup_env", "teardown_env", "get_workspace", "allreduce_rms", "allreduce_rms_fp8", "allreduce_rms_pinned",
    "fused_allreduce_rms",
    "reduce_scatter_rms", "CommProcess", "CommWorkspace", "allreduce_rms_fusion_impl", "get_comm",
    "local_workspaces", "stats", "check_status", "reference", "config", "Config", "ALGO_CODES", "OUT_SAME",
    "OUT_FP8_TOKEN", "OUT_FP8_BLOCK128",
]
