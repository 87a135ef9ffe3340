"""Shared benchmark plumbing: process-group bootstrap from torchrun's environment, device-side
timing with rank alignment and L2 flushing, max-over-ranks reduction, and loading of the
reference build for the comparison arm."""
from __future__ import annotations

import os
import statistics
import sys
import time
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(REPO, "baseline", "_ref")


def init_dist(n_gpus: int):
    """Returns (rank, world, local_rank). Uses torchrun's env; a single process needs no group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n_gpus:
        if world == 1 and n_gpus > 1:
            raise SystemExit(f"--gpus {n_gpus} needs torchrun: python -m torch.distributed.run --nnodes=1 "
                             f"--nproc-per-node {n_gpus} --master-addr 127.0.0.1 --master-port <P> bench.py --gpus {n_gpus} ...")
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {n_gpus}")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    return rank, world, local


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def min_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return float(t.item())


class RankAligner:
    """Device-side alignment of the ranks before a timed launch (a tiny NCCL all-reduce)."""

    def __init__(self, world: int):
        self.world = world
        self.t = torch.zeros(1, device="cuda") if world > 1 else None

    def __call__(self):
        if self.world > 1:
            dist.all_reduce(self.t)


HEAD_START_CYCLES = 400_000   # ~0.2 ms of device-side delay


def device_times_us(fn: Callable[[], None], steps: int, warmup: int, flush: Optional[Callable[[], None]],
                    align: Callable[[], None]) -> List[float]:
    """Per-step device time in microseconds: CUDA events around `fn` only; before every step the
    L2 is flushed (if given) and the ranks are aligned on the device. A short device-side delay
    precedes the first event so that the host has queued the whole step before the GPU reaches
    it: the interval then holds device work only, not Python launch latency. The alignment comes
    last, so that differing clocks during the delay do not skew the ranks."""
    for _ in range(warmup):
        if flush:
            flush()
        align()
        fn()
    torch.cuda.synchronize()
    pairs = []
    for _ in range(steps):
        if flush:
            flush()
        torch.cuda._sleep(HEAD_START_CYCLES)
        align()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    return [a.elapsed_time(b) * 1e3 for a, b in pairs]


def region_time_us(fn: Callable[[], None], steps: int, warmup: int, align: Callable[[], None]) -> float:
    """Device time per step of `steps` back-to-back calls of `fn`, timed as ONE region with two CUDA
    events. `fn` must rotate over inputs that together exceed the L2. The stream is first held
    back by a device-side delay sized from the measured host cost of a call, so that the whole
    region is queued before the GPU starts it and no host launch latency is inside the interval;
    the ranks are aligned after the delay."""
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    probe = min(steps, 20)
    for _ in range(probe):
        fn()
    host_s = (time.perf_counter() - t0) / probe      # host-side cost of one call (GPU keeps up or not)
    torch.cuda.synchronize()
    clock_hz = 2.0e9
    cycles = int(min(max(1.5 * host_s * steps, 2e-4), 0.25) * clock_hz)
    torch.cuda._sleep(cycles)
    align()
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / steps


def pipelined_us(fn: Callable[[], None], calls: int, warmup: int, align: Callable[[], None]) -> float:
    """Average device time per call when `calls` launches are queued back to back."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    align()
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(calls):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / calls


def barrier(world: int):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def load_reference():
    """Imports the reference package from baseline/_ref (built from its unmodified sources).

    Returns (module, None) or (None, reason)."""
    lib = os.path.join(REF_DIR, "libtorch_dist_ext.so")
    dev = os.path.join(REF_DIR, "libtorch_dist_ext_device.so")
    if not (os.path.exists(lib) and os.path.exists(dev)):
        return None, "reference build not present under baseline/_ref (offline install failed or was not run)"
    if "torch_dist_ext_b200" in sys.modules:
        return None, "the reference registers the same op namespace as this library; use a separate process"
    try:
        sys.path.insert(0, REF_DIR)
        import io
        from contextlib import redirect_stdout

        with redirect_stdout(io.StringIO()):  # the reference prints its library path on import
            import torch_dist_ext as ref_mod
        return ref_mod, None
    except Exception as e:  # pragma: no cover
        return None, f"reference import failed: {type(e).__name__}: {e}"


def timing_utils():
    """utils/timing.py loaded by path, so that the reference arm can use the clock sampler and the
    L2 flusher without importing this library's package (which would register its ops)."""
    import importlib.util

    path = os.path.join(REPO, "torch_dist_ext_b200", "utils", "timing.py")
    spec = importlib.util.spec_from_file_location("_tdx_timing", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def out_dir() -> str:
    """Directory for benchmark JSON: $TDX_OUT_DIR, else the first existing scratch directory, else bench_out/."""
    d = os.environ.get("TDX_OUT_DIR")
    if not d:
        cands = [c for c in sorted(os.listdir(REPO)) if c.endswith("_out") and os.path.isdir(os.path.join(REPO, c))]
        d = os.path.join(REPO, cands[0]) if cands else os.path.join(REPO, "bench_out")
    os.makedirs(d, exist_ok=True)
    return d


def summarize(us: List[float]) -> dict:
    s = sorted(us)
    return {"mean": statistics.fmean(us), "median": statistics.median(us), "min": s[0],
            "p90": s[min(len(s) - 1, int(0.9 * len(s)))]}


def now() -> float:
    return time.perf_counter()
