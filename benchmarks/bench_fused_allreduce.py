#!/usr/bin/env python
"""Latency sweep of the fused all-reduce + residual + RMSNorm (+ fp8 quant) op.

    python -m torch.distributed.run --nproc-per-node N benchmarks/bench_fused_allreduce.py --gpus N
        [--impl own|reference] [--quick] [--out <dir>/sweep_tpN.json]

For every (tokens, hidden) it times, on the device and as the maximum over ranks:
  own arm        every algorithm (one-shot Lamport, two-shot Lamport, two-shot flag barrier,
                 NVLS one-shot / two-shot when a multicast mapping exists), the automatic choice,
                 the fp8 per-token and 1x128 block-scaled epilogues, and the baseline
                 "NCCL all-reduce + separate residual/RMSNorm kernel (+ separate quant kernel)";
  reference arm  the reference build's op (no fp8: the reference has none).
Each figure is the time per call of a region of back-to-back calls that rotate over more than
160 MiB of inputs (see benchmarks/common.py: region_time_us). Also derives the measured
one-shot / two-shot crossover per rank count, which can be fed back through TDX_POLICY_JSON.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from benchmarks import common  # noqa: E402

EPS = 1e-6


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--out", default=None)
    ap.add_argument("--tokens", default=None, help="comma-separated token counts (default: the full sweep)")
    ap.add_argument("--hidden", default=None, help="comma-separated hidden sizes for the bf16 part")
    ap.add_argument("--no-fp8", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        cur = os.environ.get("LD_LIBRARY_PATH", "")
        if common.REF_DIR not in cur.split(":"):
            os.environ["LD_LIBRARY_PATH"] = common.REF_DIR + (":" + cur if cur else "")
            os.execve(sys.executable, [sys.executable] + sys.argv, os.environ)
    rank, world, local = common.init_dist(args.gpus)
    align = common.RankAligner(world)
    tokens_list = [1, 8, 32, 128, 512, 2048, 8192]
    hidden_list = [4096, 8192]
    fp8_hidden = [5120, 7168]
    if args.quick:
        tokens_list, fp8_hidden = [1, 128, 2048], [7168]
    if args.tokens:
        tokens_list = [int(t) for t in args.tokens.split(",")]
    if args.hidden:
        hidden_list = [int(t) for t in args.hidden.split(",")]
    if args.no_fp8:
        fp8_hidden = []

    if args.impl == "reference":
        api, why = common.load_reference()
        if api is None or world not in (2, 4, 8):
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": why or "the reference needs 2, 4 or 8 ranks"}))
            return
        api.setup_env(rank, world)
    else:
        import torch_dist_ext_b200 as api
        from torch_dist_ext_b200.ops import norm as norm_ops, quant as quant_ops
        from torch_dist_ext_b200.utils.config import OUT_FP8_BLOCK128, OUT_FP8_TOKEN

        api.setup_env(rank, world, device=local)
    import torch.distributed as dist

    rows = []

    def inputs(tokens, hidden):
        per = 2 * tokens * hidden * 2
        n = max(2, min(64, (160 << 20) // per + 1))
        g = torch.Generator().manual_seed(7 + rank)
        xs = [torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).cuda() for _ in range(min(n, 8))]
        xs = [xs[i % len(xs)].clone() for i in range(n)]
        rs = [torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
        gamma = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
        return xs, rs, gamma

    def timed(fn, steps):
        return round(common.max_over_ranks(common.region_time_us(fn, steps, 3, align), world), 2)

    for hidden in hidden_list + fp8_hidden:
        for tokens in tokens_list:
            msg = tokens * hidden * 2
            steps = args.steps if msg <= (8 << 20) else max(10, args.steps // 4)
            xs, rs, gamma = inputs(tokens, hidden)
            st = {"i": 0}

            def rot():
                st["i"] = (st["i"] + 1) % len(xs)
                return xs[st["i"]], rs[st["i"]]

            row = {"tokens": tokens, "hidden": hidden, "bytes": msg, "tp": world}
            if args.impl == "reference":
                ws = api.get_workspace(xs[0])
                common.barrier(world)
                threads = hidden // 8
                if threads > 1024 or (threads == 1024 and world >= 4):
                    # 1024-thread blocks need <= 64 registers; the reference's bf16 kernels use 79-105
                    # at 4 and 8 ranks, so its cooperative launch fails (and the failure is ignored).
                    row["reference_us"] = "n/a: launch cannot be resident (registers x 1024 threads)"
                elif hidden in fp8_hidden and False:
                    pass
                else:
                    out = api.allreduce_rms(rank, world, xs[0], rs[0], gamma, EPS, ws)
                    torch.cuda.synchronize()
                    # The reference ignores the result of its cooperative launch; a launch that cannot be
                    # resident leaves the outputs unwritten and "runs" in no time. Check against NCCL + PyTorch.
                    ref_sum = xs[0].float().clone()
                    dist.all_reduce(ref_sum)
                    e_res = (ref_sum.to(torch.bfloat16).float() + rs[0].float()).to(torch.bfloat16).float()
                    e_norm = e_res * torch.rsqrt(e_res.pow(2).mean(-1, keepdim=True) + EPS) * gamma.float()
                    ok = bool(torch.isfinite(out[0].float()).all()) and \
                        (out[0].float() - e_norm).abs().max().item() <= 0.06 * max(1.0, e_norm.abs().max().item())
                    ok = bool(common.min_over_ranks(1.0 if ok else 0.0, world))
                    if ok:
                        row["reference_us"] = timed(lambda: api.allreduce_rms(rank, world, *rot(), gamma, EPS, ws), steps)
                    else:
                        row["reference_us"] = "n/a: outputs wrong or unwritten (its cooperative launch failed and the error is ignored)"
                rows.append(row)
                continue
            if hidden in hidden_list:
                algos = ["auto"] if world == 1 else ["oneshot", "twoshot", "twoshot_barrier"]
                if world > 1 and api.stats().get("has_multicast"):
                    algos += ["oneshot_mc", "twoshot_mc", "nvls_oneshot", "nvls_twoshot"]
                if world > 1:
                    algos += ["auto"]
                for algo in algos:
                    try:
                        row[algo] = timed(lambda: api.fused_allreduce_rms(*rot(), gamma, EPS, algo=None if algo == "auto" else algo), steps)
                    except RuntimeError as e:
                        row[algo] = None
                if world > 1:
                    buf = torch.zeros_like(xs[0])

                    def nccl_sep():
                        dist.all_reduce(buf)
                        norm_ops.fused_add_rmsnorm(buf, rot()[1], gamma, EPS)

                    row["nccl_plus_kernel"] = timed(nccl_sep, steps)
            else:
                for name, mode in (("fp8_token", OUT_FP8_TOKEN), ("fp8_block128", OUT_FP8_BLOCK128)):
                    row[name] = timed(lambda: api.fused_allreduce_rms(*rot(), gamma, EPS, out_mode=mode), steps)
                row["bf16_out"] = timed(lambda: api.fused_allreduce_rms(*rot(), gamma, EPS), steps)
                if world > 1:
                    buf = torch.zeros_like(xs[0])

                    def nccl_sep_quant():
                        dist.all_reduce(buf)
                        n, _, _ = norm_ops.fused_add_rmsnorm(buf, rot()[1], gamma, EPS)
                        quant_ops.quant_fp8(n, block_scaled=True)

                    row["nccl_plus_norm_plus_quant_kernels"] = timed(nccl_sep_quant, steps)
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            del xs, rs
            torch.cuda.empty_cache()

    result = {"impl": args.impl, "tp": world, "rows": rows}
    if args.impl == "own" and world > 1:
        # measured crossover: largest message for which one-shot is not slower than two-shot
        one = [r["bytes"] for r in rows if r.get("oneshot") and r.get("twoshot") and r["oneshot"] <= r["twoshot"]]
        lam = [r["bytes"] for r in rows if r.get("twoshot") and r.get("twoshot_barrier") and r["twoshot"] <= r["twoshot_barrier"]]
        def best(r, *names):
            vals = [r[n] for n in names if r.get(n)]
            return min(vals) if vals else None

        # the same crossovers with the multicast-push variants taken into account, and whether those win
        one = [r["bytes"] for r in rows if best(r, "oneshot", "oneshot_mc") and best(r, "twoshot", "twoshot_mc")
               and best(r, "oneshot", "oneshot_mc") <= best(r, "twoshot", "twoshot_mc")]
        small = [r for r in rows if r["bytes"] <= (4 << 20)]
        mc1 = sum(1 if r["oneshot_mc"] < r["oneshot"] else -1 for r in small if r.get("oneshot_mc") and r.get("oneshot"))
        mc2 = sum(1 if r["twoshot_mc"] < r["twoshot"] else -1 for r in small if r.get("twoshot_mc") and r.get("twoshot"))
        p2p = [best(r, "twoshot", "twoshot_mc", "twoshot_barrier") for r in rows]
        nvls = [r["bytes"] for r, b in zip(rows, p2p) if r.get("nvls_twoshot") and b and r["nvls_twoshot"] < b]
        result["policy"] = {str(world): {"oneshot_max_bytes": max(one) if one else 0,
                                         "lamport_max_bytes": max(lam) if lam else 0,
                                         "mc_oneshot": int(mc1 > 0), "mc_twoshot": int(mc2 > 0),
                                         "nvls_min_bytes": min(nvls) if nvls else (1 << 62)}}
        result["pdl"] = bool(torch.ops.torch_dist_ext.pdl_enabled())
        result["stats"] = {k: v for k, v in api.stats().items() if k != "status"}
    if rank == 0:
        out = args.out or os.path.join(common.out_dir(), f"sweep_{args.impl}_tp{world}.json")
        os.makedirs(os.path.dirname(out) or ".", exist_ok=True)
        with open(out, "w") as f:
            json.dump(result, f, indent=1)
        print("wrote", out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
