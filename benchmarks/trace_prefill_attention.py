#!/usr/bin/env python
"""Per-role timeline of the prompt attention kernel, from inside the kernel (tracing flavour of the library).

    TDX_TRACE=1 python benchmarks/trace_prefill_attention.py [--seq 2048] [--heads 8] [--kv-heads 1]

The block with the most key chunks of head 0 stamps clock64 at fixed points of every chunk: the score issuer of the
chunk (loop top, waits passed, MMAs and commits issued), its P*V issuer (waits passed, issued) and thread 0 of the two
softmax groups (scores ready, loaded, row maximum done, probability tile free, probabilities stored, arrived). The
script prints the stamps of a few chunks and the median cycle counts per phase, and writes everything as JSON. No
profiler is involved; the stamps of one SM share one clock.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import common  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=1)
    args = ap.parse_args()
    from torch_dist_ext_b200 import _lib
    from torch_dist_ext_b200.ops import attention

    s_len, hq, hkv = args.seq, args.heads, args.kv_heads
    qkv = torch.randn(s_len, (hq + 2 * hkv) * 128, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : hq * 128].view(s_len, hq, 128)
    k = qkv[:, hq * 128: (hq + hkv) * 128].view(s_len, hkv, 128)
    v = qkv[:, (hq + hkv) * 128:].view(s_len, hkv, 128)
    for _ in range(3):
        attention.prefill_attention(q, k, v)
    torch.cuda.synchronize()
    p = _lib.ops().attention_prefill_probe()          # [3 roles, 64 chunks, 8 slots]
    n = min(64, (s_len + 127) // 128 * 2)              # chunks of the last query block
    t0 = int(p[0, 0, 0])
    rel = (p - t0).tolist()
    names_issue = ["score: loop top", "score: waits passed", "score: issued", "pv: waits passed", "pv: issued"]
    names_group = ["scores ready", "loaded", "maximum done", "tile free", "probabilities stored", "arrived"]
    print(f"last query block of head 0: {n} chunks of 64 keys; cycles since the first stamp")
    for c in list(range(0, min(4, n))) + list(range(max(4, n - 4), n)):
        print(f"chunk {c:2d}  issuers {rel[0][c][:5]}  group {c & 1} {rel[1 + (c & 1)][c][:6]}")
    steady = range(8, n - 2) if n > 12 else range(n)

    def med(values):
        values = list(values)
        return int(statistics.median(values)) if values else None

    out = {
        "chunks": n,
        "period_per_chunk": med(rel[0][c + 1][3] - rel[0][c][3] for c in steady if c + 1 < n),
        "score_issue": med(rel[0][c][2] - rel[0][c][1] for c in steady),
        "score_wait": med(rel[0][c][1] - rel[0][c][0] for c in steady),
        "pv_issue": med(rel[0][c][4] - rel[0][c][3] for c in steady),
        "group_load_and_max": med(rel[1 + (c & 1)][c][2] - rel[1 + (c & 1)][c][0] for c in steady),
        "group_turn_and_exponentials": med(rel[1 + (c & 1)][c][4] - rel[1 + (c & 1)][c][3] for c in steady),
        "group_cycle_per_own_chunk": med(rel[1 + (c & 1)][c + 2][0] - rel[1 + (c & 1)][c][0] for c in steady if c + 2 < n),
        "total_cycles": rel[0][n - 1][4],
    }
    print(json.dumps(out))
    path = os.path.join(common.out_dir(), "trace_prefill_attention.json")
    with open(path, "w") as f:
        json.dump({"summary": out, "issuer_slots": names_issue, "group_slots": names_group, "stamps": rel}, f)
    print("wrote", path)


if __name__ == "__main__":
    main()
