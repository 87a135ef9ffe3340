#!/usr/bin/env python
"""Phase timings of the fused all-reduce kernels on real ranks (tracing flavour of the library).

    TDX_TRACE=1 python -m torch.distributed.run --nproc-per-node N benchmarks/trace_fused_allreduce.py --gpus N
        [--tokens 128] [--hidden 4096] [--algos oneshot,twoshot,...] [--calls 20]

For every algorithm it runs a region of `--calls` back-to-back calls, queued ahead of the GPU with the ranks
aligned on the device (rotating inputs larger than L2), and reports, for the LAST of them and for every rank, when the blocks passed each phase of the protocol (microseconds since the block
started; minimum / median / maximum over blocks). The difference between "pushed" and "gathered" on the receiving
side is the cost of one hop through NVSwitch including the skew between the ranks. Needs the `_C_trace.so`
flavour (`python -m torch_dist_ext_b200._build --trace`).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from benchmarks import common  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--algos", default="oneshot,oneshot_mc,twoshot,twoshot_mc")
    ap.add_argument("--calls", type=int, default=40)
    args = ap.parse_args()
    rank, world, local = common.init_dist(args.gpus)
    import torch.distributed as dist

    import torch_dist_ext_b200 as tdx
    from torch_dist_ext_b200.utils.tracing import PhaseTrace

    tdx.setup_env(rank, world, device=local)
    if not torch.ops.torch_dist_ext.tracing_build():
        raise SystemExit("this script needs the tracing flavour: set TDX_TRACE=1 (and build with --trace)")
    trace = PhaseTrace(tdx.get_comm())
    align = common.RankAligner(world)
    n = max(2, (160 << 20) // (2 * args.tokens * args.hidden * 2) + 1)
    xs = [torch.randn(args.tokens, args.hidden, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    rs = [torch.randn(args.tokens, args.hidden, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    gamma = torch.ones(args.hidden, device="cuda", dtype=torch.bfloat16)
    result = {"rank": rank, "world": world, "tokens": args.tokens, "hidden": args.hidden, "algos": {}}
    for algo in args.algos.split(","):
        if world == 1:
            algo = "auto"
        try:
            for i in range(5):
                tdx.fused_allreduce_rms(xs[i % n], rs[i % n], gamma, 1e-6, algo=None if algo == "auto" else algo)
        except RuntimeError as e:
            result["algos"][algo] = {"unavailable": str(e).splitlines()[0]}
            continue
        torch.cuda.synchronize()
        common.barrier(world)
        trace.clear()
        st = {"i": 0}

        def call():
            st["i"] = (st["i"] + 1) % n
            tdx.fused_allreduce_rms(xs[st["i"]], rs[st["i"]], gamma, 1e-6, algo=None if algo == "auto" else algo)

        # the calls are queued behind a device-side delay and the ranks aligned on the device, as in the sweep:
        # the trace then shows the last call of a region in which no rank waits for its host
        per_call = common.max_over_ranks(common.region_time_us(call, args.calls, 3, align), world)
        result["algos"][algo] = dict(trace.summary(), region_us_per_call=round(per_call, 2))
        tdx.check_status()
        if world == 1:
            break
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, result)
    else:
        gathered = [result]
    if rank == 0:
        path = os.path.join(common.out_dir(), f"trace_tp{world}_{args.tokens}x{args.hidden}.json")
        with open(path, "w") as f:
            json.dump(gathered, f, indent=1)
        for algo, s in gathered[0]["algos"].items():
            print(algo, json.dumps(s))
        print("wrote", path)
    trace.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
