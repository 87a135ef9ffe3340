"""Greedy sampling over a vocabulary that is sharded across tensor-parallel ranks.

The reference has no sampler: its op ends at the normalised hidden state (src/ops/all_reduce_fusion.cpp:10-56).
A served model needs one, and with a sharded lm-head the step used to be ``max`` + ``stack`` + an NCCL all-gather +
``argmax`` + fancy indexing. Here it is two small kernels around one call of the fused all-reduce: every rank writes
its candidate {logit, index} into its slot of an otherwise zero row, the SUM over ranks gathers the candidates (the
all-reduce adds zeros, so the values arrive exact), and a second kernel picks the winner. No NCCL call is left in a
captured decode step.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..utils.tracing import traced
from . import reference as _ref


@traced("tdx.greedy_sample_sharded")
def greedy_sample_sharded(logits: torch.Tensor, rank: int, world: int, index_base: int) -> torch.Tensor:
    """``logits`` fp32 [tokens, vocab_shard] of this rank -> int64 [tokens]: the arg-max over the whole vocabulary.

    ``index_base`` is the vocabulary index of this shard's first column. Of equal logits the lowest index wins on
    every rank, so all ranks return the same tokens.
    """
    tokens = logits.shape[0]
    if not logits.is_cuda:
        return _ref.greedy_sample_sharded(logits, rank, world, index_base)
    ops = _lib.ops()
    pack = torch.empty(tokens, 4 * world, dtype=torch.float32, device=logits.device)
    ops.argmax_pack(logits, index_base, rank, world, pack)
    if world > 1:
        from .fused_allreduce import fused_allreduce_rms
        ones = _ones(4 * world, logits.device)
        _, pack, _ = fused_allreduce_rms(pack, None, ones, 1e-6)
    out = torch.empty(tokens, dtype=torch.int64, device=logits.device)
    ops.select_token(pack, world, out)
    return out


_ONES = {}


def _ones(n: int, device: torch.device) -> torch.Tensor:
    key = (n, device)
    if key not in _ONES:
        _ONES[key] = torch.ones(n, dtype=torch.float32, device=device)
    return _ONES[key]
