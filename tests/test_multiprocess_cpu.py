"""Process-level plumbing on CPU ranks (gloo, world_size 2): setup_env, get_workspace and the
public op run end to end against the single-process oracle, and host-side failures surface as
errors instead of hangs. No GPU is involved.

BASELINE config: per rank input [128, 4096] fp32 ~N(0,1) seeded by rank, residual with a shared
seed, weight ~N(1, 0.1), eps 1e-6; outputs: summed residual stream, normalised output, and the
fp8 e4m3 per-token quantisation with fp32 scales [128, 1].
"""
import socket
from datetime import timedelta

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dist_worker import worker
from torch_dist_ext_b200.utils.config import OUT_FP8_BLOCK128, OUT_FP8_TOKEN, OUT_SAME


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_world(world, backend, cases, target=worker):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, backend, cases, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(world):
            r = q.get(timeout=300)
            results.append(r)
            if r[1] != "ok":
                break       # the other ranks may now be stuck in a collective: do not wait for them
    except Exception:
        pass
    bad = [r for r in results if r[1] != "ok"]
    for p in procs:
        p.join(timeout=5 if bad or len(results) < world else 60)
    for p in procs:
        if p.is_alive():
            p.terminate()       # exactly the processes this test started
            p.join(timeout=10)
    assert not bad, "\n".join(str(b[2]) for b in bad)
    assert len(results) == world, f"only {len(results)} of {world} ranks reported within the time limit"
    return results


def test_gloo_world2_fused_op_matches_oracle():
    cases = [
        (128, 4096, torch.float32, None, OUT_SAME),
        (128, 4096, torch.float32, None, OUT_FP8_TOKEN),
        (16, 1024, torch.bfloat16, None, OUT_SAME),
        (16, 1024, torch.bfloat16, None, OUT_FP8_BLOCK128),
    ]
    run_world(2, "gloo", cases)


def _never_joins(rank, world, port, q):
    """Rank 1 exits before registration; rank 0 must get an error, not a hang."""
    import torch_dist_ext_b200 as tdx

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=timedelta(seconds=5))
    if rank == 1:
        q.put((rank, "left"))
        return  # never calls setup_env
    try:
        tdx.setup_env(rank, world)
        q.put((rank, "no-error"))
    except Exception as e:  # the collective inside registration fails once the peer is gone / times out
        q.put((rank, "error:" + type(e).__name__))


def test_rank_that_never_registers_is_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_never_joins, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert got[1] == "left"
    assert got[0].startswith("error"), got
