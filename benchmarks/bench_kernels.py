#!/usr/bin/env python
"""Single-GPU roofline table of the library's kernels (no communication).

    python benchmarks/bench_kernels.py [--group gemm|gemm_prefill|gemm_one_tile|gemm_pair|gemm_persist|gemm_fp8|attention|attention_simt|attention_prefill_tc|elementwise|decode_epilogues|attention_splits|all] [--steps 30]

Every case is timed as one region of back-to-back calls between two CUDA events; the calls rotate
over enough copies of the large operand that no call finds it in the 126 MB L2. Each row reports
the time, the achieved bandwidth and FLOP rate, their fractions of the measured peaks (a STREAM-style
copy and a cuBLAS bf16 GEMM; read from MEASURED_PEAKS.json beside the repo's bench.py when present,
else an earlier measurement of the same machine type, and the row says which), and the time of the
library call that does the same work (cuBLAS through torch.matmul, PyTorch's attention and
elementwise kernels) for comparison.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from benchmarks import common  # noqa: E402

L2_BYTES = 126 << 20


def peaks():
    path = os.path.join(common.REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def rotating(make, nbytes: int):
    """Copies of an operand such that consecutive calls touch different memory (> 2 x L2 in total)."""
    n = max(2, math.ceil(2 * L2_BYTES / max(nbytes, 1)) + 1)
    return [make() for _ in range(min(n, 64))]


def time_us(fn_of_i, n_sets: int, steps: int) -> float:
    state = {"i": 0}

    def step():
        state["i"] = (state["i"] + 1) % n_sets
        fn_of_i(state["i"])

    return common.region_time_us(step, steps, 3, lambda: None)


def row(name, us, lib_us, nbytes, flops, hbm, tf, src):
    gbs = nbytes / us / 1e3
    tfl = flops / us / 1e6
    return {"case": name, "us": round(us, 2), "library_us": None if lib_us is None else round(lib_us, 2),
            "GB/s": round(gbs, 1), f"frac_hbm_of_{src}": round(gbs / hbm, 3),
            "TFLOP/s": round(tfl, 1), f"frac_bf16_of_{src}": round(tfl / tf, 3)}


def gemm_cases(dev, steps, shapes, ms, out, cta_pair=None, persistent=None):
    from torch_dist_ext_b200.ops import gemm

    hbm, tf, src = peaks()
    for (n, k) in shapes:
        ws = rotating(lambda: torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02, n * k * 2)
        for m in ms:
            a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
            if m >= 256:   # the tiled kernels against the one-tile-per-CTA kernel before timing them
                want = gemm.linear(a, ws[0], cta_pair=False, persistent=False).float()
                err = (gemm.linear(a, ws[0], cta_pair=cta_pair, persistent=persistent).float() - want).abs().max().item()
                # one bf16 rounding step of the largest output: the kernels add the K blocks in different orders
                if err > 2.0 ** -7 * max(1.0, want.abs().max().item()) or gemm.pipeline_status() != 0:
                    raise SystemExit(f"opt-in GEMM disagrees with the default kernel (max err {err}, status {gemm.pipeline_status()})")
            us = time_us(lambda i: gemm.linear(a, ws[i], cta_pair=cta_pair, persistent=persistent), len(ws), steps)
            lib = time_us(lambda i: torch.matmul(a, ws[i].t()), len(ws), steps)
            nbytes = (n * k + m * k + m * n) * 2
            tag = ("gemm bf16 (CTA pairs)" if cta_pair else "gemm bf16 (persistent)" if persistent else
                   "gemm bf16 (one tile per CTA)" if persistent is False and cta_pair is False else "gemm bf16")
            out.append(row(f"{tag} m={m} n={n} k={k}", us, lib, nbytes, 2.0 * m * n * k, hbm, tf, src))
            print(out[-1], flush=True)
        del ws
        torch.cuda.empty_cache()


def gemm_fp8_cases(dev, steps, out):
    from torch_dist_ext_b200.ops import gemm, quant

    hbm, tf, src = peaks()
    for (n, k) in [(28672, 8192), (8192, 28672)]:
        w = torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05
        wq, wscale = gemm.quantize_weight_block128(w)
        del w
        wqs = [wq] + [wq.clone() for _ in range(max(1, math.ceil(2 * L2_BYTES / (n * k))))]
        for m in (16, 64, 2048):
            a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
            aq, ascale = quant.quant_fp8(a, block_scaled=True)
            us = time_us(lambda i: gemm.linear_fp8_blockscaled(aq, ascale, wqs[i], wscale), len(wqs), steps)
            nbytes = n * k + m * k + m * n * 2
            out.append(row(f"gemm fp8 block-scaled m={m} n={n} k={k}", us, None, nbytes, 2.0 * m * n * k, hbm, 2 * tf, src))
            print(out[-1], flush=True)
        del wqs, wq
        torch.cuda.empty_cache()


def attention_cases(dev, steps, out, tensor_cores=True):
    from torch_dist_ext_b200.ops import attention

    hbm, tf, src = peaks()
    for batch in (1, 16, 64):
        length, hq, hkv, d = 2048, 32, 8, 128
        kv_bytes = 2 * batch * length * hkv * d * 2
        sets = rotating(lambda: (torch.randn(batch, length, hkv, d, device=dev, dtype=torch.bfloat16),
                                 torch.randn(batch, length, hkv, d, device=dev, dtype=torch.bfloat16)), kv_bytes)
        q = torch.randn(batch, hq, d, device=dev, dtype=torch.bfloat16)
        lens = torch.full((batch,), length, device=dev, dtype=torch.int32)
        if tensor_cores:   # a new kernel: check it before timing it
            a = attention.decode_attention(q, sets[0][0], sets[0][1], lens, length, tensor_cores=True).float()
            r = attention.decode_attention(q, sets[0][0], sets[0][1], lens, length, tensor_cores=False).float()
            if not (a - r).abs().max().item() <= 3e-2:
                raise SystemExit("tensor-core decode attention disagrees with the SIMT kernel")
        us = time_us(lambda i: attention.decode_attention(q, sets[i][0], sets[i][1], lens, length, tensor_cores=tensor_cores),
                     len(sets), steps)

        def sdpa(i):
            k, v = sets[i]
            torch.nn.functional.scaled_dot_product_attention(
                q.unsqueeze(2), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), enable_gqa=True)

        lib = time_us(sdpa, len(sets), steps)
        tag = "decode attention (tcgen05)" if tensor_cores else "decode attention"
        out.append(row(f"{tag} batch={batch} len={length} hq={hq} hkv={hkv}", us, lib, kv_bytes,
                       4.0 * batch * hq * length * d, hbm, tf, src))
        print(out[-1], flush=True)
        del sets
        torch.cuda.empty_cache()


def prefill_attention_cases(dev, steps, out):
    """Causal attention over one prompt: this library's tcgen05 kernel against PyTorch's SDPA."""
    from torch_dist_ext_b200.ops import attention

    hbm, tf, src = peaks()
    for s_len, hq, hkv in [(2048, 32, 8), (8192, 32, 8), (2048, 8, 1)]:
        qkv = torch.randn(s_len, (hq + 2 * hkv) * 128, device=dev, dtype=torch.bfloat16)
        q = qkv[:, : hq * 128].view(s_len, hq, 128)
        k = qkv[:, hq * 128: (hq + hkv) * 128].view(s_len, hkv, 128)
        v = qkv[:, (hq + hkv) * 128:].view(s_len, hkv, 128)
        got = attention.prefill_attention(q, k, v).float()

        def sdpa(_i=0):
            return torch.nn.functional.scaled_dot_product_attention(
                q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0), v.transpose(0, 1).unsqueeze(0),
                is_causal=True, enable_gqa=True).squeeze(0).transpose(0, 1)

        if not (got - sdpa().float()).abs().max().item() <= 3e-2:
            raise SystemExit("tensor-core prefill attention disagrees with scaled_dot_product_attention")
        us = time_us(lambda i: attention.prefill_attention(q, k, v), 1, steps)
        lib = time_us(sdpa, 1, steps)
        flops = 4.0 * hq * 128 * s_len * s_len / 2          # causal: half of the score matrix
        out.append(row(f"prefill attention (tcgen05) s={s_len} hq={hq} hkv={hkv}", us, lib, qkv.numel() * 2 + s_len * hq * 256,
                       flops, hbm, tf, src))
        print(out[-1], flush=True)


def elementwise_cases(dev, steps, out):
    from torch_dist_ext_b200.ops import activation, norm, quant

    hbm, tf, src = peaks()
    rows, hidden = 8192, 8192
    nb = rows * hidden * 2
    xs = rotating(lambda: torch.randn(rows, hidden, device=dev, dtype=torch.bfloat16), nb)
    r = torch.randn(rows, hidden, device=dev, dtype=torch.bfloat16)
    g = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
    us = time_us(lambda i: norm.fused_add_rmsnorm(xs[i], r, g, 1e-6), len(xs), steps)

    def torch_norm(i):
        y = xs[i] + r
        torch.nn.functional.rms_norm(y, (hidden,), g, 1e-6)

    out.append(row("residual add + rmsnorm 8192x8192 bf16", us, time_us(torch_norm, len(xs), steps), 4 * nb, 0, hbm, tf, src))
    print(out[-1], flush=True)
    us = time_us(lambda i: quant.quant_fp8(xs[i]), len(xs), steps)
    out.append(row("fp8 per-token quant 8192x8192", us, None, nb + nb // 2, 0, hbm, tf, src))
    print(out[-1], flush=True)
    us = time_us(lambda i: quant.quant_fp8(xs[i], block_scaled=True), len(xs), steps)
    out.append(row("fp8 1x128 quant 8192x8192", us, None, nb + nb // 2, 0, hbm, tf, src))
    print(out[-1], flush=True)
    us = time_us(lambda i: activation.silu_mul(xs[i]), len(xs), steps)

    def torch_silu(i):
        a, b = xs[i].chunk(2, dim=-1)
        torch.nn.functional.silu(a) * b

    out.append(row("silu(gate)*up 8192x(2x4096)", us, time_us(torch_silu, len(xs), steps), nb + nb // 2, 0, hbm, tf, src))
    print(out[-1], flush=True)
    del xs
    torch.cuda.empty_cache()
    # greedy sampling: arg-max over fp32 logits (decode batch x the vocabulary shard of a rank, and the whole vocabulary)
    from torch_dist_ext_b200.ops import sampling

    for tokens, vocab in [(16, 16032), (64, 16032), (64, 128256)]:
        lb = tokens * vocab * 4
        ls = rotating(lambda: torch.randn(tokens, vocab, device=dev), lb)
        us = time_us(lambda i: sampling.greedy_sample_sharded(ls[i], 0, 1, 0), len(ls), steps)
        out.append(row(f"arg-max over logits {tokens}x{vocab} fp32", us, time_us(lambda i: ls[i].argmax(dim=-1), len(ls), steps), lb, 0,
                       hbm, tf, src))
        print(out[-1], flush=True)
        del ls


def attention_split_cases(dev, steps, out):
    """Decode attention over the KV split count at 2048 positions (the data behind `ops/attention.py: pick_splits`)."""
    from torch_dist_ext_b200.ops import attention

    length = 2048
    for (b, hq, hkv) in [(1, 4, 1), (16, 4, 1), (64, 4, 1), (64, 8, 1), (16, 32, 8)]:
        per_set = 2 * b * length * hkv * 128 * 2
        sets = [(torch.randn(b, length, hkv, 128, device=dev, dtype=torch.bfloat16),
                 torch.randn(b, length, hkv, 128, device=dev, dtype=torch.bfloat16))
                for _ in range(max(2, min(16, (300 << 20) // per_set)))]
        q = torch.randn(b, hq, 128, device=dev, dtype=torch.bfloat16)
        lens = torch.full((b,), length, device=dev, dtype=torch.int32)
        res = {"case": f"decode attention {b} sequences x {hq} heads on {hkv} KV heads x {length}",
               "picked": attention.pick_splits(b, hkv, length, ctas_per_sm=1)}
        for ns in (None, 1, 2, 3, 4, 6, 8, 9, 12, 16):
            us = time_us(lambda i: attention.decode_attention(q, sets[i][0], sets[i][1], lens, length, nsplit=ns), len(sets), steps)
            res["auto_us" if ns is None else f"splits_{ns}_us"] = round(us, 2)
        out.append(res)
        print(res, flush=True)
        del sets
        torch.cuda.empty_cache()


def decode_epilogue_cases(dev, steps, out):
    """The decode GEMMs whose split-K finalizer does the next kernel's work, against the two-kernel form (column
    `library_us` here: this library's GEMM followed by its own RoPE + KV-append / SiLU kernel). Per-rank shapes of TP=8."""
    from torch_dist_ext_b200.ops import activation, gemm, rope

    hbm, tf, src = peaks()
    seq = 2304
    cos_sin = rope.build_cos_sin_cache(seq, 128, 5e5, dev)
    for name, hidden, q_heads, kv_heads, ffn in [("8B/8", 4096, 4, 1, 1792), ("70B/8", 8192, 8, 1, 3584)]:
        n_qkv = (q_heads + 2 * kv_heads) * 128
        wq = rotating(lambda: torch.randn(n_qkv, hidden, device=dev, dtype=torch.bfloat16) * 0.02, n_qkv * hidden * 2)
        wg = rotating(lambda: torch.randn(2 * ffn, hidden, device=dev, dtype=torch.bfloat16) * 0.02, 2 * ffn * hidden * 2)
        for m in (1, 16, 64):
            a = torch.randn(m, hidden, device=dev, dtype=torch.bfloat16)
            positions = torch.randint(2048, seq, (m,), device=dev)
            k_cache = torch.zeros(m, seq, kv_heads, 128, device=dev, dtype=torch.bfloat16)
            v_cache = torch.zeros_like(k_cache)

            def separate_qkv(i):
                qkv = gemm.linear(a, wq[i])
                q = qkv[:, : q_heads * 128].view(m, q_heads, 128)
                k = qkv[:, q_heads * 128: (q_heads + kv_heads) * 128].view(m, kv_heads, 128)
                v = qkv[:, (q_heads + kv_heads) * 128:].view(m, kv_heads, 128)
                rope.rope_append_kv_(q, k, v, positions, cos_sin, k_cache, v_cache)

            us = time_us(lambda i: gemm.linear_rope_kv(a, wq[i], positions, cos_sin, k_cache, v_cache, q_heads, kv_heads), len(wq), steps)
            out.append(row(f"qkv + rope + KV append, one kernel ({name}) m={m}", us, time_us(separate_qkv, len(wq), steps),
                           (n_qkv * hidden + m * hidden + m * n_qkv) * 2, 2.0 * m * n_qkv * hidden, hbm, tf, src))
            print(out[-1], flush=True)

            def separate_gate_up(i):
                activation.silu_mul(gemm.linear(a, wg[i]))

            us = time_us(lambda i: gemm.linear_silu_mul(a, wg[i]), len(wg), steps)
            out.append(row(f"gate/up + silu*mul, one kernel ({name}) m={m}", us, time_us(separate_gate_up, len(wg), steps),
                           (2 * ffn * hidden + m * hidden + m * ffn) * 2, 4.0 * m * ffn * hidden, hbm, tf, src))
            print(out[-1], flush=True)
        del wq, wg
        torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--group", default="all")
    ap.add_argument("--steps", type=int, default=30)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    import torch_dist_ext_b200  # noqa: F401  (loads the extension)

    out = []
    g = args.group
    if g in ("gemm", "all"):        # decode: weight streaming (Llama-3-8B shapes at TP=1)
        gemm_cases(dev, args.steps, [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)], (1, 16, 64), out)
    if g in ("gemm_prefill", "all"):   # the library's default for these shapes: persistent CTA pairs
        gemm_cases(dev, max(5, args.steps // 3), [(28672, 4096), (4096, 14336)], (2048, 8192), out)
        gemm_cases(dev, max(5, args.steps // 3), [(8192, 8192), (3584, 8192)], (2048,), out)   # Llama-3-70B shapes at TP=1 / TP=8
    if g == "gemm_one_tile":           # one 128 x N tile per CTA, no persistence (the decode kernel on prefill shapes)
        os.environ["TDX_GEMM_PERSIST"] = "0"
        gemm_cases(dev, max(5, args.steps // 3), [(28672, 4096), (4096, 14336), (8192, 8192)], (2048,), out, cta_pair=False,
                   persistent=False)
    if g == "gemm_pair":            # 256 x 256 tiles on persistent CTA pairs, named explicitly
        gemm_cases(dev, max(5, args.steps // 3), [(28672, 4096), (4096, 14336)], (2048, 8192), out, cta_pair=True)
    if g == "gemm_persist":         # persistent grid of single CTAs, 128 x 256 tiles, double-buffered accumulator
        gemm_cases(dev, max(5, args.steps // 3), [(28672, 4096), (4096, 14336)], (2048, 8192), out, persistent=True)
    if g in ("gemm_fp8", "all"):
        gemm_fp8_cases(dev, args.steps, out)
    if g in ("attention", "attention_tc", "all"):   # the tcgen05 decode kernel (the library's default)
        attention_cases(dev, args.steps, out, tensor_cores=True)
    if g == "attention_simt":       # the SIMT decode kernel (TDX_ATTN_TC=0), for comparison
        attention_cases(dev, args.steps, out, tensor_cores=False)
    if g in ("attention_prefill_tc", "all"):
        prefill_attention_cases(dev, max(5, args.steps // 3), out)
    if g in ("elementwise", "all"):
        elementwise_cases(dev, args.steps, out)
    if g == "attention_splits":     # decode attention over the KV split count
        attention_split_cases(dev, args.steps, out)
    if g == "decode_epilogues":     # rotary + KV append / silu inside the GEMM's finalizer against the two-kernel form
        decode_epilogue_cases(dev, args.steps, out)
    path = os.path.join(common.out_dir(), f"kernels_{g}.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
