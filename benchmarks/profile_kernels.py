#!/usr/bin/env python
"""Runs ONE kernel of the library a few times on a small case, for `ncu` captures.

    python benchmarks/profile_kernels.py --kernel gemm|gemm_fp8|gemm_prefill|attention|attention_prefill|fused_ar|gemm_ar|ag_gemm|ar_oneshot_emu|ar_twoshot_emu [--iters 4]

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
# a profiler that replays a launch saves and restores the process's device memory: keep the communication buffers
# small (the library reads this when it is imported)
os.environ.setdefault("TDX_LAMPORT_MB", "32")


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
    elif args.kernel == "ag_gemm":       # 16 tokens, [14336, 4096] (117 MB; 112 tiles, all resident as the kernel needs)
        x = torch.randn(16, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.randn(14336, 4096, device=dev, dtype=torch.bfloat16)
        fn = lambda: fused_gemm.allgather_gemm(x, w, 16)
    elif args.kernel == "gemm_prefill":  # the persistent CTA-pair kernel where it is compute-bound: 2048 x 8192 x 8192 bf16
        a = torch.randn(2048, 8192, device=dev, dtype=torch.bfloat16)
        w = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16) * 0.02
        fn = lambda: gemm.linear(a, w)
    elif args.kernel == "attention_prefill":   # causal attention over one 2048-token prompt, 8 query heads on 1 KV head
        qkv = torch.randn(2048, 10 * 128, device=dev, dtype=torch.bfloat16)
        q, k, v = qkv[:, :1024].view(2048, 8, 128), qkv[:, 1024:1152].view(2048, 1, 128), qkv[:, 1152:].view(2048, 1, 128)
        fn = lambda: attention.prefill_attention(q, k, v)
    elif args.kernel in ("ar_oneshot_emu", "ar_twoshot_emu"):
        # the multi-rank protocols with 8 ranks EMULATED inside one cooperative launch on this GPU (blockIdx.y = rank):
        # the only safe way to look at their stall reasons with a profiler. 128 x 4096 bf16 per rank; a short wait
        # budget, so that a replay artefact ends as a status code
        from torch_dist_ext_b200.utils.config import ALGO_CODES, OUT_SAME

        ws = tdx.local_workspaces(8, size_in_bytes=8 << 20, timeout_ms=200)
        ins = [torch.randn(128, 4096, device=dev, dtype=torch.bfloat16) for _ in range(8)]
        rr = torch.randn(128, 4096, device=dev, dtype=torch.bfloat16)
        g = torch.ones(4096, device=dev, dtype=torch.bfloat16)
        outs = [torch.empty_like(rr) for _ in range(8)]
        ress = [torch.empty_like(rr) for _ in range(8)]
        algo = ALGO_CODES["oneshot" if args.kernel == "ar_oneshot_emu" else "twoshot"]

        def fn():
            torch.ops.torch_dist_ext.allreduce_rms_emulated(ws, ins, [rr] * 8, g, ress, outs, [], 1e-6, OUT_SAME, algo, False)
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
    if args.kernel.endswith("_emu"):
        bad = [w.errors_seen() for w in ws]
        if any(bad):
            raise SystemExit(f"a device-side wait ran out in the emulated launch: {bad}")
    tdx.teardown_env()


if __name__ == "__main__":
    main()
