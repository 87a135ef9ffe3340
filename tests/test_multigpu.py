"""Real multi-process, multi-GPU runs: NCCL only bootstraps (handle exchange, barriers); the op
itself moves data with in-kernel peer loads/stores through IPC-mapped workspaces. Mirrors the
reference's distributed test (test/test_all_reduce_fusion.py:31-87) with assertions, more rank
counts, every algorithm and the fp8 epilogues. Skipped when fewer GPUs are visible.
"""
import pytest
import torch

from test_multiprocess_cpu import run_world
from torch_dist_ext_b200.utils.config import OUT_FP8_BLOCK128, OUT_FP8_TOKEN, OUT_SAME

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def cases():
    out = []
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for tokens in (129, 128, 1):
            out.append((tokens, 1024, dtype, None, OUT_SAME))
    for algo in ("oneshot", "twoshot", "twoshot_barrier"):
        out.append((64, 8192, torch.bfloat16, algo, OUT_SAME))
        out.append((257, 4096, torch.bfloat16, algo, OUT_FP8_TOKEN))
        out.append((37, 5120, torch.bfloat16, algo, OUT_FP8_BLOCK128))
    for algo in ("oneshot_mc", "twoshot_mc"):               # multicast pushes; skipped by the worker without multicast
        out.append((64, 8192, torch.bfloat16, algo, OUT_SAME))
        out.append((129, 1024, torch.float32, algo, OUT_SAME))
        out.append((257, 4096, torch.bfloat16, algo, OUT_FP8_TOKEN))
        out.append((37, 5120, torch.bfloat16, algo, OUT_FP8_BLOCK128))
        out.append((3, 1024, torch.float16, algo, OUT_SAME))
    for algo in ("nvls_oneshot", "nvls_twoshot"):           # skipped by the worker without multicast
        out.append((64, 8192, torch.bfloat16, algo, OUT_SAME))
        out.append((1, 4096, torch.float32, algo, OUT_SAME))
        out.append((257, 4096, torch.bfloat16, algo, OUT_FP8_TOKEN))
        out.append((300, 1024, torch.float16, algo, OUT_SAME))
    out.append((4096, 4096, torch.bfloat16, None, OUT_SAME))   # 32 MiB: NVLS two-shot or flag-barrier path
    return out


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_op_across_processes(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    results = run_world(world, "nccl", cases())
    counts = results[0][2]
    assert counts, "no algorithm statistics recorded"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gemm_fused_with_collectives_across_processes(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from dist_worker_gemm import worker as gemm_worker

    cases = [(1, 4096, 4096, False), (16, 4096, 4096, False), (64, 8192, 8192, False), (33, 2048, 1024, False),
             (16, 4096, 4096, True), (61, 2048, 2048, True),
             (600, 2048, 1024, False), (601, 2048, 1024, True)]      # more tiles than SMs: the persistent fused kernel
    run_world(world, "nccl", cases, target=gemm_worker)
