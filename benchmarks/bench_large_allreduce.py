#!/usr/bin/env python
"""Large messages (>= 32 MiB per rank): tuning sweep of the flag-synchronised two-shot paths.

    python -m torch.distributed.run --nproc-per-node N benchmarks/bench_large_allreduce.py --gpus N

For every shape it times the peer-to-peer two-shot and the NVLS two-shot with 1, 2 and 4 pipeline waves
(`TDX_WAVES`) and, for NVLS, 1 and 4 rows of switch-side sums requested together (`TDX_NVLS_BATCH`), on the
device and as the maximum over ranks, and reports each time as a fraction of the link-time floor of its
algorithm: bytes that must cross NVLink per direction (two-shot 2 (N-1)/N M, NVLS (1 + 1/N) M) divided by the
measured peer-copy bandwidth of this machine type (770 GB/s per direction; 900 GB/s nominal is reported too).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from benchmarks import common  # noqa: E402

LINK_GBS_MEASURED, LINK_GBS_NOMINAL = 770.0, 900.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--shapes", default="2048x8192,8192x4096,8192x8192")
    ap.add_argument("--steps", type=int, default=12)
    args = ap.parse_args()
    rank, world, local = common.init_dist(args.gpus)
    import torch.distributed as dist

    import torch_dist_ext_b200 as tdx

    tdx.setup_env(rank, world, device=local)
    align = common.RankAligner(world)
    has_mc = bool(tdx.stats().get("has_multicast"))
    rows = []
    for shape in args.shapes.split(","):
        tokens, hidden = (int(v) for v in shape.split("x"))
        m = tokens * hidden * 2
        n = max(2, (300 << 20) // (2 * m) + 1)
        xs = [torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
        rs = [torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
        gamma = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
        st = {"i": 0}
        floors = {"twoshot_barrier": 2 * (world - 1) / world * m, "nvls_twoshot": (1 + 1 / world) * m}
        for algo in ["twoshot_barrier"] + (["nvls_twoshot"] if has_mc else []):
            for waves in (1, 2, 4):
                for batch in ((1, 4) if algo == "nvls_twoshot" else (1,)):
                    torch.ops.torch_dist_ext.set_tuning(waves, batch)

                    def call():
                        st["i"] = (st["i"] + 1) % n
                        tdx.fused_allreduce_rms(xs[st["i"]], rs[st["i"]], gamma, 1e-6, algo=algo)

                    us = common.max_over_ranks(common.region_time_us(call, args.steps, 3, align), world)
                    tdx.check_status()
                    floor_us = floors[algo] / LINK_GBS_MEASURED / 1e3
                    row = {"tokens": tokens, "hidden": hidden, "bytes": m, "tp": world, "algo": algo, "waves": waves,
                           "nvls_batch": batch, "us": round(us, 1), "link_floor_us_at_770": round(floor_us, 1),
                           "fraction_of_floor_at_770": round(floor_us / us, 3),
                           "fraction_of_floor_at_900": round(floors[algo] / LINK_GBS_NOMINAL / 1e3 / us, 3)}
                    rows.append(row)
                    if rank == 0:
                        print(json.dumps(row), flush=True)
        torch.ops.torch_dist_ext.set_tuning(-1, -1)
        del xs, rs
        torch.cuda.empty_cache()
    if rank == 0:
        path = os.path.join(common.out_dir(), f"large_allreduce_tp{world}.json")
        with open(path, "w") as f:
            json.dump(rows, f, indent=1)
        print("wrote", path)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
