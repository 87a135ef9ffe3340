"""Llama-shaped tensor-parallel decoder built on the fused ops.

One process per GPU; every rank holds a 1/world shard of the attention heads and of the FFN.
Per layer and decode step::

    qkv   = x @ Wqkv_r^T                                  tcgen05 GEMM (column-parallel, no comm)
    q, k  = rope(q, k)  ;  cache[pos] = k, v
    attn  = split-KV decode attention over the local heads
    x,res = (attn @ Wo_r^T  --all-reduce-->) + res -> RMSNorm      tcgen05 GEMM, then ONE kernel for all-reduce +
    gu    = x @ Wgu_r^T ;  act = silu(gate) * up                   residual + norm (+ e4m3 quantisation); or both in
    x,res = (act @ Wd_r^T --all-reduce-->) + res -> RMSNorm        one kernel (GEMM -> reduce-scatter -> norm -> gather)

``mode="sp"`` keeps the normalised rows scattered (rank r owns rows r::world) and feeds them to the
next column-parallel GEMM through the fused all-gather->GEMM kernel instead (bf16 weights; with e4m3
weights the e4m3 rows and their scales are gathered by the process group and the block-scaled GEMM follows).

With ``fp8=True`` the four projection weights are e4m3 with 128x128 fp32 block scales; the
activations that feed them are quantised to e4m3 with 1x128 scales by the producing kernel
(RMSNorm epilogue, SiLU-mul) and the GEMMs promote every 128-wide K block in fp32.

The reference has no model code; this module is the serving loop that its fused op was written
for, used by the decode-throughput benchmark. Weights are random (N(0, 0.02)): there is no
checkpoint format.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import activation, attention, fused_gemm, gemm, norm, quant, rope, sampling
from ..ops.fused_allreduce import fused_allreduce_rms
from ..parallel import comm as _comm
from ..utils.config import OUT_FP8_BLOCK128, OUT_SAME
from ..utils.tracing import nvtx_range, traced

# prompt-phase attention: this library's tcgen05 kernel; "sdpa" selects PyTorch's kernel for comparisons
_PREFILL_ATTN_TC = os.environ.get("TDX_PREFILL_ATTN", "tc").lower() != "sdpa"
# Row-parallel projections (o_proj, down_proj) run as GEMM + the fused all-reduce op (two launches) by default: with
# dependent launch and the one-shot all-reduce at decode sizes that measured faster than the fused GEMM + all-reduce
# kernel, whose tail is a two-hop reduce-scatter + gather - Llama-3-8B shapes, 8 layers, batch 1 / 16 / 64: 99 / 109 /
# 161 against 112 / 122 / 191 us per layer on two B200, 80 / 83 / 117 against 94 / 97 / 148 on four; Llama-3-70B shapes
# with e4m3 weights, batch 64: 262 against 301 (two) and 171 against 213 (four).
# TDX_FUSED_BF16=1 / TDX_FUSED_FP8=1 select the fused kernel for bf16 / e4m3 weights.
_FUSED_FP8 = os.environ.get("TDX_FUSED_FP8", "0") != "0"
_FUSED_BF16 = os.environ.get("TDX_FUSED_BF16", "0") != "0"
# Decode steps in "ar" mode run the rotary embedding + KV append inside the qkv GEMM and (bf16 weights) silu(gate) * up
# inside the gate_up GEMM: both live in the GEMM's split-K finalizer and each saves a launch of the layer's latency
# chain. Measured on one B200 at the per-rank shapes of TP=8 (CUDA-graph replay of 8 layers, same box, fused against
# separate kernels): Llama-3-8B 51.3 / 55.2 against 54.3 / 59.7 us per layer at batch 1 / 16, Llama-3-70B (e4m3, rotary
# part only) 84.7 / 88.3 against 85.8 / 90.1; at batch 64 the finalizer - one CTA per 128 output features, after the
# last K split has arrived - is the longer path (100.0 against 94.5 and 137.1 against 130.9), so the fused form is used
# up to TDX_FUSED_EPILOGUE_TOKENS (16) tokens. TDX_FUSED_EPILOGUES=0 keeps the separate kernels everywhere.
_FUSED_EPILOGUES = os.environ.get("TDX_FUSED_EPILOGUES", "1") != "0"
_FUSED_EPILOGUE_TOKENS = int(os.environ.get("TDX_FUSED_EPILOGUE_TOKENS", "16"))


@dataclass
class LlamaConfig:
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    n_layers: int = 32
    vocab: int = 128256
    rope_theta: float = 5e5
    eps: float = 1e-5
    head_dim: int = 128
    fp8: bool = False

    @staticmethod
    def llama3_8b(**kw) -> "LlamaConfig":
        return LlamaConfig(**kw)

    @staticmethod
    def llama3_70b(**kw) -> "LlamaConfig":
        base = dict(hidden=8192, n_heads=64, n_kv_heads=8, ffn=28672, n_layers=80, fp8=True)
        base.update(kw)
        return LlamaConfig(**base)

    @staticmethod
    def shard_of(cfg: "LlamaConfig", tp: int, **kw) -> "LlamaConfig":
        """What ONE rank of a ``tp``-way tensor-parallel ``cfg`` computes, as a single-rank model: the same GEMM,
        attention and elementwise shapes per layer (heads and FFN divided by ``tp``, at least one KV head), with
        the collectives reduced to their local tail. For single-GPU launch lists and kernel timing of the
        tensor-parallel layer."""
        base = dict(hidden=cfg.hidden, n_heads=cfg.n_heads // tp, n_kv_heads=max(1, cfg.n_kv_heads // tp), ffn=cfg.ffn // tp,
                    n_layers=cfg.n_layers, vocab=cfg.vocab // tp, rope_theta=cfg.rope_theta, eps=cfg.eps,
                    head_dim=cfg.head_dim, fp8=cfg.fp8)
        base.update(kw)
        return LlamaConfig(**base)

    @staticmethod
    def tiny(**kw) -> "LlamaConfig":
        base = dict(hidden=512, n_heads=8, n_kv_heads=8, ffn=1024, n_layers=2, vocab=1024)
        base.update(kw)
        return LlamaConfig(**base)


class _Linear:
    """A weight shard [out, in] in bf16, or e4m3 + 128x128 block scales."""

    def __init__(self, out_f: int, in_f: int, device, gen: torch.Generator, fp8: bool):
        w = (torch.randn(out_f, in_f, device=device, generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        self.out_f, self.in_f, self.fp8 = out_f, in_f, fp8
        if fp8:
            pad = (-out_f) % 128
            if pad:
                w = torch.cat([w, w.new_zeros(pad, in_f)])
            self.w, self.scale = gemm.quantize_weight_block128(w)
        else:
            self.w, self.scale = w, None

    def __call__(self, x: torch.Tensor, x_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.fp8:
            if x_scale is None:
                x, x_scale = quant.quant_fp8(x, block_scaled=True)
            y = gemm.linear_fp8_blockscaled(x, x_scale, self.w, self.scale)
            return y[:, : self.out_f] if y.shape[1] != self.out_f else y
        return gemm.linear(x, self.w)

    def dequantized(self) -> torch.Tensor:
        if not self.fp8:
            return self.w.float()
        n, k = self.w.shape
        w = (self.w.float().view(n // 128, 128, k // 128, 128) * self.scale.view(n // 128, 1, k // 128, 1)).view(n, k)
        return w[: self.out_f]


class TPLlama:
    def __init__(self, cfg: LlamaConfig, max_batch: int, max_seq: int, mode: str = "ar", seed: int = 0,
                 device: Optional[torch.device] = None):
        c = _comm.get_comm()
        self.cfg, self.mode = cfg, mode
        self.rank, self.world, self.group = c.rank, c.world_size, c.group
        self.device = device or c.device
        assert cfg.n_heads % self.world == 0 and cfg.ffn % self.world == 0, "heads and FFN must divide by the world size"
        assert mode in ("ar", "sp")
        self.hq = cfg.n_heads // self.world
        # fewer KV heads than ranks: every rank keeps the KV head its query heads belong to
        self.hkv = max(1, cfg.n_kv_heads // self.world)
        self.ffn_r = cfg.ffn // self.world
        d = cfg.head_dim
        gen = torch.Generator(device=self.device).manual_seed(seed * 1000 + self.rank)
        gen_shared = torch.Generator(device=self.device).manual_seed(seed * 1000 + 999)
        self.embed = (torch.randn(cfg.vocab, cfg.hidden, device=self.device, generator=gen_shared) * 0.02).to(torch.bfloat16)
        vocab_r = (cfg.vocab + self.world - 1) // self.world
        self.vocab_r = vocab_r
        self.lm_head = (torch.randn(vocab_r, cfg.hidden, device=self.device, generator=gen) * 0.02).to(torch.bfloat16)
        self.layers = []
        for _ in range(cfg.n_layers):
            ones = lambda: (1.0 + 0.02 * torch.randn(cfg.hidden, device=self.device, generator=gen_shared)).to(torch.bfloat16)
            self.layers.append(dict(
                ln1=ones(), ln2=ones(),
                wqkv=_Linear((self.hq + 2 * self.hkv) * d, cfg.hidden, self.device, gen, cfg.fp8),
                wo=_Linear(cfg.hidden, self.hq * d, self.device, gen, cfg.fp8),
                wgu=_Linear(2 * self.ffn_r, cfg.hidden, self.device, gen, cfg.fp8),
                wd=_Linear(cfg.hidden, self.ffn_r, self.device, gen, cfg.fp8),
            ))
        self.final_norm = (1.0 + 0.02 * torch.randn(cfg.hidden, device=self.device, generator=gen_shared)).to(torch.bfloat16)
        self.max_batch, self.max_seq = max_batch, max_seq
        self.k_cache = [torch.zeros(max_batch, max_seq, self.hkv, d, dtype=torch.bfloat16, device=self.device)
                        for _ in range(cfg.n_layers)]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]
        self.cos_sin = rope.build_cos_sin_cache(max_seq, d, cfg.rope_theta, self.device)
        self.seq_lens = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self._graph = None
        self._static = {}

    # ---- building blocks -----------------------------------------------------------------------
    def _norm_out_mode(self) -> int:
        return OUT_FP8_BLOCK128 if self.cfg.fp8 else OUT_SAME

    def _row_parallel(self, a: torch.Tensor, lin: _Linear, res: torch.Tensor, gamma: torch.Tensor, a_scale=None):
        """a @ W_r^T -> all-reduce (or reduce-scatter) -> + res -> RMSNorm. Returns (x, x_scale, res)."""
        scatter = self.mode == "sp"
        if lin.fp8:
            # block-scaled e4m3 operands: GEMM + all-reduce op by default, the fused kernel on request (see _FUSED_FP8);
            # either way the epilogue quantises the next layer's input
            if a_scale is None:
                a, a_scale = quant.quant_fp8(a, block_scaled=True)
            x, res, xs = fused_gemm.gemm_allreduce_rms(a, lin.w, res, gamma, self.cfg.eps, out_mode=OUT_FP8_BLOCK128,
                                                       scatter_only=scatter, a_scale=a_scale, w_scale=lin.scale,
                                                       force_unfused=not _FUSED_FP8)
            return x, xs, res
        x, res, xs = fused_gemm.gemm_allreduce_rms(a, lin.w, res, gamma, self.cfg.eps, out_mode=OUT_SAME,
                                                   scatter_only=scatter, force_unfused=not _FUSED_BF16)
        return x, xs, res

    def _col_parallel(self, x: torch.Tensor, lin: _Linear, tokens: int, x_scale=None) -> torch.Tensor:
        if self.mode == "sp" and not lin.fp8:
            return fused_gemm.allgather_gemm(x, lin.w, tokens)
        if self.mode == "sp":
            # e4m3 rows and their 1x128 scales are gathered as they are (half the bytes of bf16 rows), then the
            # block-scaled GEMM runs on the full batch; the fused all-gather GEMM takes bf16 rows only
            full = self._gather_rows(x.view(torch.uint8), tokens).view(torch.float8_e4m3fn)
            return lin(full, self._gather_rows(x_scale, tokens))
        return lin(x, x_scale)

    def _layer(self, i: int, x, x_scale, res, positions, tokens: int, max_len: int, bf16_tail: bool = False):
        """One decoder layer of a decode step. ``bf16_tail`` (last layer of an fp8 model): the
        down projection is a plain GEMM followed by the all-reduce whose epilogue writes bf16,
        because the final norm feeds the bf16 lm_head."""
        cfg, L, d = self.cfg, self.layers[i], self.cfg.head_dim
        fuse = (_FUSED_EPILOGUES and self.mode == "ar" and d == 128 and tokens <= _FUSED_EPILOGUE_TOKENS
                and gemm.fused_epilogue_fits(tokens, cfg.hidden, 1 if cfg.fp8 else 2, cfg.fp8))
        if fuse:
            if cfg.fp8 and x_scale is None:
                x, x_scale = quant.quant_fp8(x, block_scaled=True)
            qkv = gemm.linear_rope_kv(x, L["wqkv"].w, positions, self.cos_sin, self.k_cache[i], self.v_cache[i], self.hq,
                                      self.hkv, a_scale=x_scale, w_scale=L["wqkv"].scale)
            q = qkv[:, : self.hq * d].view(tokens, self.hq, d)
        else:
            qkv = self._col_parallel(x, L["wqkv"], tokens, x_scale)
            q = qkv[:, : self.hq * d].view(tokens, self.hq, d)
            k = qkv[:, self.hq * d: (self.hq + self.hkv) * d].view(tokens, self.hkv, d)
            v = qkv[:, (self.hq + self.hkv) * d:].view(tokens, self.hkv, d)
            rope.rope_append_kv_(q, k, v, positions, self.cos_sin, self.k_cache[i], self.v_cache[i])
        attn = attention.decode_attention(q, self.k_cache[i][:tokens], self.v_cache[i][:tokens], self.seq_lens[:tokens], max_len)
        x, x_scale, res = self._row_parallel(attn.view(tokens, self.hq * d), L["wo"], res, L["ln2"])
        if fuse and not cfg.fp8 and self.ffn_r % 64 == 0:
            act, act_scale = gemm.linear_silu_mul(x, L["wgu"].w), None
        else:
            gu = self._col_parallel(x, L["wgu"], tokens, x_scale)
            act, act_scale = activation.silu_mul(gu, quant_block128=cfg.fp8)
        if bf16_tail:
            y = L["wd"](act, act_scale)
            x, res, _ = fused_allreduce_rms(y, res, self.final_norm, cfg.eps, out_mode=OUT_SAME, scatter_only=self.mode == "sp")
            return x, None, res
        next_gamma = self.layers[i + 1]["ln1"] if i + 1 < cfg.n_layers else self.final_norm
        return self._row_parallel(act, L["wd"], res, next_gamma, act_scale)

    def _logits_argmax(self, x: torch.Tensor, tokens: int) -> torch.Tensor:
        if self.mode == "sp":
            x = self._gather_rows(x, tokens)
        if x.dtype == torch.float8_e4m3fn:
            raise RuntimeError("final norm output must be bf16")
        logits = gemm.linear(x, self.lm_head, out_dtype=torch.float32)          # [tokens, vocab_r]
        return sampling.greedy_sample_sharded(logits, self.rank, self.world, self.rank * self.vocab_r)

    def _gather_rows(self, x_shard: torch.Tensor, tokens: int) -> torch.Tensor:
        n = self.world
        rows = (tokens + n - 1) // n
        pad = x_shard.new_zeros(rows, x_shard.shape[1])
        pad[: x_shard.shape[0]] = x_shard[:rows]
        parts = [torch.empty_like(pad) for _ in range(n)]
        if n > 1:
            dist.all_gather(parts, pad, group=self.group)
        else:
            parts = [pad]
        return torch.stack(parts, dim=1).reshape(rows * n, -1)[:tokens].contiguous()

    # ---- decode -----------------------------------------------------------------------------------
    @traced("tdx.decode_step")
    def decode_step(self, tokens: torch.Tensor, positions: torch.Tensor, max_len: int) -> torch.Tensor:
        """One token per sequence: ``tokens``/``positions`` int64 [B] on the device. Returns next tokens [B]."""
        b = tokens.shape[0]
        cfg = self.cfg
        self.seq_lens[:b] = (positions + 1).to(torch.int32)
        res = self.embed[tokens]                                                  # [B, hidden]
        mode0 = self._norm_out_mode()
        if self.mode == "sp":
            # this rank's rows (rank, rank + world, ...), padded to the common shard height so that
            # every rank - also one that owns a row less, or none - passes tensors of the same shape
            rows = (b + self.world - 1) // self.world
            shard = res[self.rank::self.world]
            if shard.shape[0] < rows:
                shard = torch.cat([shard, shard.new_zeros(rows - shard.shape[0], cfg.hidden)])
            res = shard.contiguous()
        x, _, x_scale = norm.fused_add_rmsnorm(res, None, self.layers[0]["ln1"], cfg.eps, out_mode=mode0, want_residual=False)
        for i in range(cfg.n_layers):
            last = i + 1 == cfg.n_layers
            with nvtx_range(f"tdx.layer{i}"):
                x, x_scale, res = self._layer(i, x, x_scale, res, positions, b, max_len, bf16_tail=last and cfg.fp8)
        self.last_hidden = x          # final normalised hidden state (kept for tests and probes)
        return self._logits_argmax(x, b)

    # ---- CUDA graph ------------------------------------------------------------------------------------
    def capture_decode(self, batch: int, max_len: int) -> None:
        """Capture one decode step for a fixed batch size into a CUDA graph (replayed by `decode`)."""
        st = self._static
        st["tokens"] = torch.zeros(batch, dtype=torch.long, device=self.device)
        st["positions"] = torch.zeros(batch, dtype=torch.long, device=self.device)
        st["max_len"] = max_len
        # warm-up on a side stream (allocations, lazy initialisation), then capture
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                st["out"] = self.decode_step(st["tokens"], st["positions"], max_len)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            st["out"] = self.decode_step(st["tokens"], st["positions"], max_len)
        self._graph = g

    def decode(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Replay the captured step (falls back to eager when nothing was captured)."""
        if self._graph is None:
            return self.decode_step(tokens, positions, self.max_seq)
        self._static["tokens"].copy_(tokens, non_blocking=True)
        self._static["positions"].copy_(positions, non_blocking=True)
        self._graph.replay()
        return self._static["out"]

    # ---- prefill ------------------------------------------------------------------------------------------
    def fill_cache_random(self, batch: int, length: int, seed: int = 1) -> None:
        """Synthetic context: random bf16 keys/values for `length` positions of `batch` sequences."""
        g = torch.Generator(device=self.device).manual_seed(seed + self.rank)
        for k, v in zip(self.k_cache, self.v_cache):
            k[:batch, :length] = torch.randn(batch, length, self.hkv, self.cfg.head_dim, device=self.device, generator=g).to(torch.bfloat16)
            v[:batch, :length] = torch.randn(batch, length, self.hkv, self.cfg.head_dim, device=self.device, generator=g).to(torch.bfloat16)

    @traced("tdx.prefill")
    def prefill(self, token_ids: torch.Tensor, seq_index: int = 0) -> torch.Tensor:
        """Run one prompt ``[S]`` through all layers, filling row ``seq_index`` of the KV cache.

        GEMMs and the fused all-reduce+norm run on this library's kernels (normal-orientation
        tcgen05 tiles, two-shot / NVLS all-reduce), causal attention over the prompt included
        (``TDX_PREFILL_ATTN=sdpa`` swaps in PyTorch's scaled_dot_product_attention for comparisons).
        Returns the first generated token."""
        cfg, d = self.cfg, self.cfg.head_dim
        assert self.mode == "ar", "prefill is implemented for the replicated (all-reduce) mode"
        s = token_ids.shape[0]
        positions = torch.arange(s, device=self.device)
        res = self.embed[token_ids]
        x, _, x_scale = norm.fused_add_rmsnorm(res, None, self.layers[0]["ln1"], cfg.eps, out_mode=self._norm_out_mode(), want_residual=False)
        for i, L in enumerate(self.layers):
            qkv = L["wqkv"](x, x_scale)
            q = qkv[:, : self.hq * d].view(s, self.hq, d)
            k = qkv[:, self.hq * d: (self.hq + self.hkv) * d].view(s, self.hkv, d)
            v = qkv[:, (self.hq + self.hkv) * d:].view(s, self.hkv, d)
            rope.rope_(q, k, positions, self.cos_sin)
            self.k_cache[i][seq_index, :s] = k
            self.v_cache[i][seq_index, :s] = v
            if _PREFILL_ATTN_TC:
                attn = attention.prefill_attention(q, k, v).view(s, self.hq * d)
            else:
                attn = torch.nn.functional.scaled_dot_product_attention(
                    q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0), v.transpose(0, 1).unsqueeze(0),
                    is_causal=True, enable_gqa=True).squeeze(0).transpose(0, 1).reshape(s, self.hq * d)
            y = L["wo"](attn.contiguous())
            last = i + 1 == cfg.n_layers
            x, res, x_scale = fused_allreduce_rms(y, res, L["ln2"], cfg.eps, out_mode=self._norm_out_mode())
            gu = L["wgu"](x, x_scale)
            act, act_scale = activation.silu_mul(gu, quant_block128=cfg.fp8)
            y = L["wd"](act, act_scale)
            gamma = self.layers[i + 1]["ln1"] if not last else self.final_norm
            x, res, x_scale = fused_allreduce_rms(y, res, gamma, cfg.eps, out_mode=OUT_SAME if last else self._norm_out_mode())
        return self._logits_argmax(x[-1:].contiguous(), 1)

    # ---- reference (single process, fp32, PyTorch only) ---------------------------------------------------------
    def weights_for_reference(self) -> dict:
        """Dequantised shards of this rank, for the PyTorch oracle used by the tests."""
        return dict(layers=[{k: (v.dequantized() if isinstance(v, _Linear) else v.float()) for k, v in L.items()}
                            for L in self.layers],
                    embed=self.embed.float(), lm_head=self.lm_head.float(), final_norm=self.final_norm.float())
