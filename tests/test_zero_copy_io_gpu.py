"""The fused op on data that stays in pinned host memory (`allreduce_rms_pinned`).

The kernels are the ones the device-tensor path launches; only the addresses differ (the inputs are
read and the outputs written over PCIe by the kernel itself). Checked here on one GPU: the
single-rank call through the public API, the multi-rank protocols with all ranks emulated in one
cooperative launch and every data tensor in pinned memory, and the rejection of pageable memory
before anything is launched. The reference has no such entry point (its op takes device tensors
only, src/ops/all_reduce_fusion.cpp:14-61).
"""
import pytest
import torch

import torch_dist_ext_b200 as tdx
from helpers import check_against_oracle
from torch_dist_ext_b200.utils.config import ALGO_CODES, OUT_SAME

pytestmark = pytest.mark.gpu
EPS = 1e-6


@pytest.fixture(scope="module")
def workspaces():
    cache = {}

    def get(n):
        if n not in cache:
            cache[n] = tdx.local_workspaces(n, size_in_bytes=8 << 20, timeout_ms=2000)
        return cache[n]

    yield get
    torch.cuda.synchronize()
    cache.clear()


def _pinned_inputs(nranks, tokens, hidden, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    ins = [torch.randn(tokens, hidden, generator=g).to(dtype).pin_memory() for _ in range(nranks)]
    residual = torch.randn(tokens, hidden, generator=g).to(dtype).pin_memory()
    gamma = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).cuda()
    return ins, residual, gamma


def test_single_rank_public_api_matches_device_path():
    tdx.setup_env(0, 1)
    for dtype in (torch.bfloat16, torch.float32):
        (x,), r, gamma = _pinned_inputs(1, 33, 2048, dtype, seed=5)
        out = (torch.zeros_like(x).pin_memory(), torch.zeros_like(x).pin_memory())
        norm, res = tdx.allreduce_rms_pinned(x, r, gamma, EPS, out=out)
        torch.cuda.synchronize()
        assert norm.data_ptr() == out[0].data_ptr() and not norm.is_cuda
        d_norm, d_res = tdx.allreduce_rms(0, 1, x.cuda(), r.cuda(), gamma, EPS, tdx.get_workspace(gamma))
        torch.cuda.synchronize()
        assert torch.equal(norm, d_norm.cpu()) and torch.equal(res, d_res.cpu())
    tdx.check_status()


@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "twoshot_barrier"])
@pytest.mark.parametrize("nranks", [2, 8])
def test_emulated_ranks_with_every_tensor_in_pinned_memory(workspaces, nranks, algo):
    ws = workspaces(nranks)
    for tokens, hidden in [(3, 1024), (130, 1024), (17, 4096)]:
        ins, residual, gamma = _pinned_inputs(nranks, tokens, hidden, torch.bfloat16, seed=tokens)
        norm = [torch.zeros(tokens, hidden, dtype=torch.bfloat16).pin_memory() for _ in range(nranks)]
        res = [torch.zeros(tokens, hidden, dtype=torch.bfloat16).pin_memory() for _ in range(nranks)]
        for repeat in range(3):                      # the Lamport buffers rotate over three calls
            used = torch.ops.torch_dist_ext.allreduce_rms_emulated(
                ws, ins, [residual] * nranks, gamma, res, norm, [], EPS, OUT_SAME, ALGO_CODES[algo], False)
            torch.cuda.synchronize()
            assert used == ALGO_CODES[algo]
            check_against_oracle([t.cuda() for t in ins], residual.cuda(), gamma, EPS, OUT_SAME,
                                 [t.cuda() for t in norm], [t.cuda() for t in res], [])
    assert all(w.errors_seen() == 0 for w in ws)
    torch.cuda.synchronize()


def test_pageable_memory_is_rejected_before_launch():
    tdx.setup_env(0, 1)
    (x,), r, gamma = _pinned_inputs(1, 4, 1024, torch.bfloat16, seed=1)
    pageable = torch.empty(x.shape, dtype=x.dtype).copy_(x)
    with pytest.raises(RuntimeError, match="pinned"):
        tdx.allreduce_rms_pinned(pageable, r, gamma, EPS, out=(torch.zeros_like(x).pin_memory(), torch.zeros_like(x).pin_memory()))
    torch.cuda.synchronize()
    tdx.check_status()
