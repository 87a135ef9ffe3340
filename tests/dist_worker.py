"""Worker run by every rank of the multi-process tests (gloo on CPU, NCCL + real IPC on GPUs)."""
from __future__ import annotations

import os
import sys
import traceback

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_case(world, tokens, hidden, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    ins = [torch.randn(tokens, hidden, generator=g).to(dtype) for _ in range(world)]
    residual = torch.randn(tokens, hidden, generator=g).to(dtype)
    gamma = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    return ins, residual, gamma


def worker(rank: int, world: int, port: int, backend: str, cases, result_queue=None):
    """Runs `cases` = [(tokens, hidden, dtype, algo, out_mode)] and asserts against the oracle."""
    try:
        import torch_dist_ext_b200 as tdx
        from torch_dist_ext_b200.utils.config import OUT_SAME

        cuda = backend == "nccl"
        if cuda:
            torch.cuda.set_device(rank)
        dist.init_process_group(backend=backend, init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        tdx.setup_env(rank, world, max_size_in_bytes=32 << 20)
        dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
        tol = {torch.float32: 2e-5, torch.float16: 4e-3, torch.bfloat16: 3.2e-2}
        has_mc = cuda and tdx.stats().get("has_multicast", False)
        for i, (tokens, hidden, dtype, algo, out_mode) in enumerate(cases):
            nvls = isinstance(algo, str) and algo.startswith("nvls")
            if (nvls or (isinstance(algo, str) and algo.endswith("_mc"))) and not has_mc:
                continue
            # the automatic choice moves large messages onto the NVLS path when there is one
            nvls_min = {2: 1 << 62, 4: 1 << 62}.get(world, 12 << 20)
            nvls = nvls or (algo is None and has_mc and tokens * hidden * torch.finfo(dtype).bits // 8 >= nvls_min)
            ins, residual, gamma = make_case(world, tokens, hidden, dtype, seed=i)
            exp_norm, exp_res, exp_scale = tdx.reference.fused_allreduce_rms_reference(ins, residual, gamma, 1e-6, out_mode)
            x, r, w = ins[rank].to(dev), residual.to(dev), gamma.to(dev)
            if out_mode == OUT_SAME and algo is None:
                ws = tdx.get_workspace(x)
                norm, res = tdx.allreduce_rms(rank, world, x, r, w, 1e-6, ws)
                scales = None
            else:
                norm, res, scales = tdx.fused_allreduce_rms(x, r, w, 1e-6, out_mode=out_mode, algo=algo)
            if cuda:
                torch.cuda.synchronize()
                tdx.check_status()
            if nvls:
                # The switch accumulates in fp32 but rounds the sum to the element type in its own way
                # (results one step below round-to-nearest were observed), so the sum s may differ by one
                # step of ITS magnitude; that error then passes unchanged through the residual add.
                step = {torch.float32: 2.0 ** -22, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}[dtype]
                sabs = sum(t.float().abs() for t in ins)
                d = (res.cpu().float() - exp_res.float()).abs()
                lim = (sabs + exp_res.float().abs()) * step + 1e-6
                assert bool((d <= lim).all()), f"case {i}: NVLS residual_out off by {d.max().item()} on rank {rank}"
            else:
                assert torch.equal(res.cpu().float(), exp_res.float()), f"case {i}: residual_out mismatch on rank {rank}"
            if nvls and out_mode == OUT_SAME:
                err = (norm.cpu().float() - exp_norm.float()).abs().max().item()
                assert err <= 4 * tol[dtype] * max(1.0, exp_norm.float().abs().max().item()), f"case {i}: NVLS norm err {err}"
            elif nvls:
                back = tdx.reference.dequantize_fp8(norm.cpu(), scales.cpu())
                want = tdx.reference.dequantize_fp8(exp_norm, exp_scale)
                assert (back - want).abs().max().item() <= want.abs().max().item() * 2.0 ** -3, f"case {i}: NVLS fp8"
            elif out_mode == OUT_SAME:
                err = (norm.cpu().float() - exp_norm.float()).abs().max().item()
                assert err <= tol[dtype] * max(1.0, exp_norm.float().abs().max().item()), f"case {i}: norm err {err}"
            else:
                assert torch.allclose(scales.cpu(), exp_scale, rtol=1e-5), f"case {i}: scales mismatch"
                got, want = norm.cpu().float(), exp_norm.float()
                step = torch.maximum(got.abs(), want.abs()) * 0.125 + 2.0 ** -9
                assert bool(((got - want).abs() <= step).all()), f"case {i}: fp8 codes differ by more than a step"
            if cuda and out_mode == OUT_SAME and not nvls and algo in (None, "oneshot", "twoshot", "twoshot_barrier"):
                # the same call on pinned host tensors: the peer-to-peer paths are deterministic, so the kernel
                # that reads and writes host memory itself must reproduce the device-tensor result bit for bit
                outs = (torch.zeros(tokens, hidden, dtype=dtype).pin_memory(), torch.zeros(tokens, hidden, dtype=dtype).pin_memory())
                p_norm, p_res = tdx.allreduce_rms_pinned(ins[rank].pin_memory(), residual.pin_memory(), w, 1e-6, out=outs, algo=algo)
                torch.cuda.synchronize()
                tdx.check_status()
                assert torch.equal(p_res, res.cpu()) and torch.equal(p_norm, norm.cpu()), f"case {i}: pinned-memory path differs on rank {rank}"
        # greedy sampling over a sharded vocabulary: the candidates are gathered by the fused all-reduce itself
        from torch_dist_ext_b200.ops import sampling
        g = torch.Generator().manual_seed(4242)
        full = torch.randn(33, world * 1000, generator=g)
        full[5, 17] = full[5, world * 1000 - 3] = 9.0          # equal logits in the first and the last shard: the lower index wins
        want = full.argmax(dim=-1)
        want[5] = 17
        mine = full[:, rank * 1000:(rank + 1) * 1000].contiguous().to(dev)
        got = sampling.greedy_sample_sharded(mine, rank, world, rank * 1000)
        if cuda:
            torch.cuda.synchronize()
            tdx.check_status()
        assert torch.equal(got.cpu(), want), f"sharded greedy sampling differs on rank {rank}"
        st = tdx.stats()
        if cuda:
            assert st["error_count"] == 0
        dist.barrier()
        tdx.teardown_env()
        dist.destroy_process_group()
        if result_queue is not None:
            result_queue.put((rank, "ok", dict(st.get("algo_counts") or {}, has_multicast=bool(st.get("has_multicast")))))
    except Exception:
        if result_queue is not None:
            result_queue.put((rank, "error", traceback.format_exc()))
        raise
