"""Tiny end-to-end check used by the driver's smoke run: one decode step of a 2-layer
Llama-shaped model on a single GPU (bf16 and fp8 weights)."""
from __future__ import annotations

import torch

from .. import setup_env, teardown_env
from .llama import LlamaConfig, TPLlama


def run(device) -> None:
    setup_env(0, 1, max_size_in_bytes=8 << 20)
    try:
        for fp8 in (False, True):
            model = TPLlama(LlamaConfig.tiny(fp8=fp8), max_batch=4, max_seq=64, device=device)
            model.fill_cache_random(4, 16)
            tokens = torch.randint(0, 1024, (4,), device=device)
            positions = torch.full((4,), 16, device=device, dtype=torch.long)
            nxt = model.decode_step(tokens, positions, max_len=17)
            torch.cuda.synchronize()
            assert nxt.shape == (4,) and bool((nxt >= 0).all()) and bool((nxt < 1024).all())
            assert bool(torch.isfinite(model.last_hidden.float()).all())
    finally:
        teardown_env()
