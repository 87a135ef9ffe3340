"""Worker of the multi-GPU tests of the GEMM+collective kernels and the tensor-parallel layer."""
from __future__ import annotations

import os
import sys
import traceback

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def worker(rank: int, world: int, port: int, backend: str, cases, result_queue=None):
    try:
        import torch_dist_ext_b200 as tdx
        from torch_dist_ext_b200.ops import fused_gemm, gemm
        from torch_dist_ext_b200.ops import reference as ref

        torch.cuda.set_device(rank)
        dist.init_process_group(backend=backend, init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        tdx.setup_env(rank, world, max_size_in_bytes=32 << 20)
        dev = torch.device("cuda", rank)
        for i, (tokens, hidden, k_total, scatter) in enumerate(cases):
            g = torch.Generator().manual_seed(100 + i)
            a_full = torch.randn(tokens, k_total, generator=g).to(torch.bfloat16)
            w_full = (torch.randn(hidden, k_total, generator=g) * 0.05).to(torch.bfloat16)
            residual = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
            gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
            ks = k_total // world
            parts = [(a_full[:, r * ks:(r + 1) * ks].float() @ w_full[:, r * ks:(r + 1) * ks].float().t()).to(torch.bfloat16)
                     for r in range(world)]
            e_norm, e_res, _ = ref.fused_allreduce_rms_reference(parts, residual, gamma, 1e-6)
            a = a_full[:, rank * ks:(rank + 1) * ks].contiguous().to(dev)
            w = w_full[:, rank * ks:(rank + 1) * ks].contiguous().to(dev)
            if scatter:   # ragged tail: the last ranks own one row less; pad to the common shard shape
                rows = (tokens + world - 1) // world
                res_in = torch.zeros(rows, hidden, dtype=torch.bfloat16)
                part = residual[rank::world]
                res_in[: part.shape[0]] = part
                res_in = res_in.to(dev)
            else:
                res_in = residual.to(dev)
            # replicated output: both tails of the fused kernel (one hop / two hops), then the op's own choice
            for hop in ((True, False, None) if not scatter else (None,)):
                for _ in range(3):
                    norm, res, _ = fused_gemm.gemm_allreduce_rms(a, w, res_in, gamma.to(dev), 1e-6, scatter_only=scatter, one_hop=hop)
                torch.cuda.synchronize()
                tdx.check_status()
                kk0 = (e_norm[rank::world] if scatter else e_norm).shape[0]
                want0 = e_res[rank::world] if scatter else e_res
                assert (res[:kk0].cpu().float() - want0.float()).abs().max().item() <= 0.13, f"case {i} (one_hop={hop}): residual"
            torch.cuda.synchronize()
            tdx.check_status()
            want_n = e_norm[rank::world] if scatter else e_norm
            want_r = e_res[rank::world] if scatter else e_res
            kk = want_n.shape[0]
            assert (res[:kk].cpu().float() - want_r.float()).abs().max().item() <= 0.13, f"case {i}: residual"
            assert (norm[:kk].cpu().float() - want_n.float()).abs().max().item() <= 0.13, f"case {i}: norm"
            # all-gather -> GEMM on the scattered norm rows
            if scatter:
                w2 = (torch.randn(256, hidden, generator=g) * 0.05).to(torch.bfloat16)
                for _ in range(3):
                    out = fused_gemm.allgather_gemm(norm[:kk].contiguous(), w2.to(dev), tokens)
                torch.cuda.synchronize()
                tdx.check_status()
                # gather the reference from what every rank holds: use the oracle's norm
                want = e_norm.float() @ w2.float().t()
                err = (out.cpu().float() - want).abs().max().item()
                assert err <= 0.05 * want.abs().max().item() + 0.05, f"case {i}: ag_gemm err {err}"
        # tensor-parallel model: replicated (all-reduce) and sequence-parallel modes agree
        from torch_dist_ext_b200.models.llama import LlamaConfig, TPLlama

        hidden_states = {}
        nb = {2: 6, 4: 8}.get(world, 2 * world)      # sequences in the batch
        for mode in ("ar", "sp"):
            model = TPLlama(LlamaConfig.tiny(), max_batch=nb, max_seq=64, mode=mode, seed=3)
            model.fill_cache_random(nb, 12, seed=5)
            tokens = torch.arange(nb, device=dev) * 7 % 1024
            positions = torch.full((nb,), 12, device=dev, dtype=torch.long)
            nxt = model.decode_step(tokens, positions, max_len=13)
            torch.cuda.synchronize()
            tdx.check_status()
            h = model.last_hidden.float()
            hidden_states[mode] = model._gather_rows(model.last_hidden, nb).float() if mode == "sp" else h
            allt = [torch.empty_like(nxt) for _ in range(world)]
            dist.all_gather(allt, nxt)
            assert all(torch.equal(t, nxt) for t in allt), "ranks disagree on the next tokens"
            del model
        diff = (hidden_states["ar"] - hidden_states["sp"]).abs().max().item()
        assert diff <= 0.08, f"replicated and sequence-parallel modes differ by {diff}"
        # the same pair of modes with e4m3 weights: the scattered rows travel as e4m3 with their 1x128 scales
        hs = {}
        for mode in ("ar", "sp"):
            model = TPLlama(LlamaConfig.tiny(fp8=True), max_batch=nb, max_seq=64, mode=mode, seed=3)
            model.fill_cache_random(nb, 12, seed=5)
            model.decode_step(tokens, positions, max_len=13)
            torch.cuda.synchronize()
            tdx.check_status()
            hs[mode] = model._gather_rows(model.last_hidden, nb).float() if mode == "sp" else model.last_hidden.float()
            del model
        diff = (hs["ar"] - hs["sp"]).abs().max().item()
        assert diff <= 0.15, f"e4m3 weights: replicated and sequence-parallel modes differ by {diff}"
        assert gemm.pipeline_status() == 0
        dist.barrier()
        tdx.teardown_env()
        dist.destroy_process_group()
        if result_queue is not None:
            result_queue.put((rank, "ok", None))
    except Exception:
        if result_queue is not None:
            result_queue.put((rank, "error", traceback.format_exc()))
        raise
