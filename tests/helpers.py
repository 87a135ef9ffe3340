"""Shared helpers for the kernel tests: inputs, oracle comparison, emulated multi-rank calls."""
from __future__ import annotations

import torch

import torch_dist_ext_b200  # noqa: F401  (loads the library)
from torch_dist_ext_b200.ops import reference as ref
from torch_dist_ext_b200.utils.config import ALGO_CODES, OUT_FP8_TOKEN, OUT_SAME

TOL = {torch.float32: 2e-5, torch.float16: 4e-3, torch.bfloat16: 3.2e-2}


def make_inputs(nranks, tokens, hidden, dtype, device, seed=0, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    ins = [(torch.randn(tokens, hidden, generator=g) * scale).to(dtype).to(device) for _ in range(nranks)]
    residual = torch.randn(tokens, hidden, generator=g).to(dtype).to(device)
    gamma = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).to(device)
    return ins, residual, gamma


def run_emulated(ws, ins, residual, gamma, eps, out_mode, algo, scatter_only=False):
    n = len(ins)
    tokens, hidden = ins[0].shape
    dev = ins[0].device
    rows = (tokens + n - 1) // n if scatter_only else tokens
    def shard(t, r):
        part = t[r::n]
        if part.shape[0] < rows:  # ragged tail: the last ranks own one row less; pad to the common shape
            part = torch.cat([part, part.new_zeros(rows - part.shape[0], hidden)])
        return part.contiguous()

    res_in = [shard(residual, r) if scatter_only else residual for r in range(n)]
    res_out = [torch.full((rows, hidden), float("nan"), dtype=ins[0].dtype, device=dev) for _ in range(n)]
    if out_mode == OUT_SAME:
        norm = [torch.full((rows, hidden), float("nan"), dtype=ins[0].dtype, device=dev) for _ in range(n)]
        scales = []
    else:
        norm = [torch.zeros(rows, hidden, dtype=torch.float8_e4m3fn, device=dev) for _ in range(n)]
        ncol = 1 if out_mode == OUT_FP8_TOKEN else hidden // 128
        scales = [torch.full((rows, ncol), float("nan"), dtype=torch.float32, device=dev) for _ in range(n)]
    used = torch.ops.torch_dist_ext.allreduce_rms_emulated(ws, ins, res_in, gamma, res_out, norm, scales, eps,
                                                           out_mode, ALGO_CODES[algo], scatter_only)
    torch.cuda.synchronize()
    return used, norm, res_out, scales


def check_against_oracle(ins, residual, gamma, eps, out_mode, norm, res_out, scales, scatter_only=False):
    n = len(ins)
    dtype = ins[0].dtype
    exp_norm, exp_res, exp_scale = ref.fused_allreduce_rms_reference(ins, residual, gamma, eps, out_mode)
    tol = TOL[dtype]
    for r in range(n):
        e_res = exp_res[r::n] if scatter_only else exp_res
        # the residual stream is an exact function of the inputs: fp32 sum in rank order, two roundings
        assert torch.equal(res_out[r].float(), e_res.float()), f"rank {r}: residual_out differs"
        if out_mode == OUT_SAME:
            e_norm = exp_norm[r::n] if scatter_only else exp_norm
            err = (norm[r].float() - e_norm.float()).abs().max().item()
            assert err <= tol * max(1.0, e_norm.float().abs().max().item()), f"rank {r}: norm_out max err {err}"
        else:
            e_scale = exp_scale[r::n] if scatter_only else exp_scale
            e_q = exp_norm[r::n] if scatter_only else exp_norm
            assert torch.allclose(scales[r], e_scale, rtol=1e-5, atol=1e-12), f"rank {r}: scales differ"
            # compare the e4m3 codes as numbers: at most one code step apart (ulp <= |v|/8, or
            # 2^-9 in the subnormal range), which is what a last-bit difference in rsqrt can cause
            got, want = norm[r].float(), e_q.float()
            step = torch.maximum(got.abs(), want.abs()) * 0.125 + 2.0 ** -9
            assert bool(((got - want).abs() <= step).all()), f"rank {r}: fp8 output off by more than one code step"
            frac_diff = (norm[r].view(torch.uint8) != e_q.view(torch.uint8)).float().mean().item()
            assert frac_diff < 0.02, f"rank {r}: {frac_diff:.3%} of fp8 codes differ from the oracle"
    for r in range(1, n):
        if not scatter_only:
            assert torch.equal(norm[r].view(torch.uint8), norm[0].view(torch.uint8)), "ranks disagree bitwise"
