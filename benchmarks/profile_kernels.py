#!/usr/bin/env python
"""Runs ONE kernel of the library a few times on a small case, for `ncu` captures.

    python benchmarks/profile_kernels.py --kernel gemm|gemm_fp8|attention|fused_ar|gemm_ar|ag_gemm [--iters 4]

Cases are sized so that the inputs exceed the 126 MB L2 where the kernel is bandwidth-bound, while
the process holds well under a few GB, so that a multi-pass `ncu --set full` capture of one to three
launches ends by itself in about a minute. Single GPU: the collective kernels run with this rank as
its own only peer (the full code path, local memory).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True)
    ap.add_argument("--iters", type=int, default=4)
    args = ap.parse_args()
    import torch_dist_ext_b200 as tdx
    from torch_dist_ext_b200.ops import attention, fused_gemm, gemm, quant

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tdx.setup_env(0, 1, max_size_in_bytes=16 << 20)
    if args.kernel == "gemm":            # decode-shaped weight streaming: 16 tokens x [28672, 4096] bf16 (235 MB)
        a = torch.randn(16, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.randn(28672, 4096, device=dev, dtype=torch.bfloat16)
        fn = lambda: gemm.linear(a, w)
    elif args.kernel == "gemm_fp8":      # block-scaled e4m3: 16 tokens x [28672, 8192] (235 MB)
        a = torch.randn(16, 8192, device=dev, dtype=torch.bfloat16)
        w = torch.randn(28672, 8192, device=dev, dtype=torch.bfloat16) * 0.05
        aq, as_ = quant.quant_fp8(a, block_scaled=True)
        wq, ws_ = gemm.quantize_weight_block128(w)
        del w
        fn = lambda: gemm.linear_fp8_blockscaled(aq, as_, wq, ws_)
    elif args.kernel == "attention":     # 16 sequences x 2048 positions x 8 KV heads (134 MB of K+V), G = 4
        q = torch.randn(16, 32, 128, device=dev, dtype=torch.bfloat16)
        k = torch.randn(16, 2048, 8, 128, device=dev, dtype=torch.bfloat16)
        v = torch.randn_like(k)
        lens = torch.full((16,), 2048, device=dev, dtype=torch.int32)
        fn = lambda: attention.decode_attention(q, k, v, lens, 2048)
    elif args.kernel == "fused_ar":      # residual + RMSNorm epilogue path, 8192 x 8192 bf16 (128 MiB per tensor)
        x = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
        r = torch.randn_like(x)
        g = torch.ones(8192, device=dev, dtype=torch.bfloat16)
        fn = lambda: tdx.fused_allreduce_rms(x, r, g, 1e-6)
    elif args.kernel == "gemm_ar":       # down_proj-shaped: 16 tokens, hidden 4096, K 14336 (117 MB of weights)
        a = torch.randn(16, 14336, device=dev, dtype=torch.bfloat16)
        w = torch.randn(4096, 14336, device=dev, dtype=torch.bfloat16) * 0.02
        r = torch.randn(16, 4096, device=dev, dtype=torch.bfloat16)
        g = torch.ones(4096, device=dev, dtype=torch.bfloat16)
        fn = lambda: fused_gemm.gemm_allreduce_rms(a, w, r, g, 1e-6)
    elif args.kernel == "ag_gemm":       # gate_up-shaped: 16 tokens, [28672, 4096]
        x = torch.randn(16, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.randn(28672, 4096, device=dev, dtype=torch.bfloat16)
        fn = lambda: fused_gemm.allgather_gemm(x, w, 16)
    else:
        raise SystemExit(f"unknown kernel {args.kernel}")
    for _ in range(args.iters):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    print(f"{args.kernel}: last call {e0.elapsed_time(e1) * 1e3:.1f} us (CUDA events)")
    tdx.teardown_env()


if __name__ == "__main__":
    main()
