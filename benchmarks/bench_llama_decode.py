#!/usr/bin/env python
"""Decode throughput of Llama-shaped tensor-parallel models on this library's kernels.

    python -m torch.distributed.run --nproc-per-node N benchmarks/bench_llama_decode.py --gpus N
        --model 8b|70b|tiny|8b-shard8|70b-shard8 [--layers L] [--batch 1,16,64] [--kv 2048] [--steps 128] [--mode ar|sp]

Weights are random (N(0, 0.02)); the KV cache is filled with random bf16 for `--kv` positions per
sequence (`--prefill` instead runs one real `--kv`-token prompt per sequence through the prefill
path first, times it, and adds prefill tokens/s and the end-to-end generated tokens/s of both
phases). One decode step = one new token for every sequence of the batch, replayed from a CUDA
graph; the timed region holds `--steps` steps between two CUDA events, maximum over ranks.
Reports microseconds per step and per layer, tokens/s for the whole job, and the weight-streaming
floor (weight bytes per rank / measured HBM copy bandwidth).
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
    ap.add_argument("--model", default="8b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", default="1,16,64")
    ap.add_argument("--kv", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--mode", default="ar")
    ap.add_argument("--prefill", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    rank, world, local = common.init_dist(args.gpus)
    import torch_dist_ext_b200 as tdx
    from torch_dist_ext_b200.models.llama import LlamaConfig, TPLlama

    tdx.setup_env(rank, world, max_size_in_bytes=64 << 20, device=local)
    if args.model.endswith("-shard8"):
        # one rank's share of the TP=8 model, run as a single-rank model (kernel shapes of the TP=8 layer on one GPU)
        full = {"8b": LlamaConfig.llama3_8b, "70b": LlamaConfig.llama3_70b}[args.model[:-7]]()
        cfg = LlamaConfig.shard_of(full, 8)
    else:
        cfg = {"8b": LlamaConfig.llama3_8b, "70b": LlamaConfig.llama3_70b, "tiny": LlamaConfig.tiny}[args.model]()
    if args.layers:
        cfg.n_layers = args.layers
    batches = [int(b) for b in args.batch.split(",")]
    max_batch = max(batches)
    model = TPLlama(cfg, max_batch=max_batch, max_seq=args.kv + args.steps + 8, mode=args.mode)
    align = common.RankAligner(world)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(common.REPO, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = peaks.get("hbm_gbs", 6650.0) * 1e9
    wbytes = sum(sum(t.numel() * t.element_size() for t in (L[k].w,)) for L in model.layers for k in ("wqkv", "wo", "wgu", "wd"))
    rows = []
    for b in batches:
        prefill_ms = None
        if args.prefill:
            prompts = [torch.randint(0, cfg.vocab, (args.kv,), device=model.device) for _ in range(b)]
            torch.cuda.synchronize()
            common.barrier(world)
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record()
            for s in range(b):
                model.prefill(prompts[s], seq_index=s)
            p1.record()
            torch.cuda.synchronize()
            prefill_ms = common.max_over_ranks(p0.elapsed_time(p1), world)
        else:
            model.fill_cache_random(b, args.kv)
        tokens = torch.randint(0, cfg.vocab, (b,), device=model.device)
        pos = torch.full((b,), args.kv, device=model.device, dtype=torch.long)
        if not args.no_graph:
            model.capture_decode(b, max_len=args.kv + args.steps + 1)
        state = {"tokens": tokens, "pos": pos.clone()}

        def step():
            state["tokens"] = model.decode(state["tokens"], state["pos"]) if not args.no_graph else \
                model.decode_step(state["tokens"], state["pos"], args.kv + args.steps + 1)
            state["pos"] += 1

        for _ in range(3):
            step()
        state["pos"].copy_(pos)
        torch.cuda.synchronize()
        common.barrier(world)
        align()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        us = common.max_over_ranks(e0.elapsed_time(e1) * 1e3 / args.steps, world)
        kv_bytes = 2 * cfg.n_layers * b * (args.kv + args.steps // 2) * model.hkv * cfg.head_dim * 2
        floor_us = (wbytes + kv_bytes) / hbm * 1e6
        tdx.check_status()
        row = {"model": args.model, "layers": cfg.n_layers, "tp": world, "mode": args.mode, "fp8": cfg.fp8, "batch": b,
               "kv_len": args.kv, "steps": args.steps, "us_per_step": round(us, 1), "us_per_layer": round(us / cfg.n_layers, 2),
               "tokens_per_s": round(b / us * 1e6, 1), "weight_bytes_per_rank": wbytes,
               "hbm_floor_us_per_step": round(floor_us, 1), "fraction_of_hbm_floor": round(floor_us / us, 3),
               "cuda_graph": not args.no_graph}
        if prefill_ms is not None:
            # prompt processing + generation, as one job: generated tokens over the time of both phases
            total_s = prefill_ms / 1e3 + us * args.steps / 1e6
            row.update({"prefill_ms": round(prefill_ms, 2), "prefill_tokens_per_s": round(b * args.kv / prefill_ms * 1e3, 1),
                        "end_to_end_generated_tokens_per_s": round(b * args.steps / total_s, 1)})
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        model._graph = None
    if rank == 0:
        out = args.out or os.path.join(common.out_dir(), f"llama_{args.model}_tp{world}_{args.mode}.json")
        os.makedirs(os.path.dirname(out) or ".", exist_ok=True)
        json.dump(rows, open(out, "w"), indent=1)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
