"""Runs the standalone C++ harness (no PyTorch in the process): the reference's shape sweep in
fp32 plus bf16 cases, every algorithm, with a non-zero exit code on any mismatch."""
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu
BIN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp", "unit_test.bin")


def run(args):
    assert os.path.exists(BIN), "build the harness first: python -m torch_dist_ext_b200._build"
    res = subprocess.run([BIN] + args, capture_output=True, text=True, timeout=900)
    tail = "\n".join(res.stdout.splitlines()[-15:]) + res.stderr[-2000:]
    assert res.returncode == 0, tail
    assert "result:PASS" in res.stdout, tail


def test_four_ranks_emulated_on_one_gpu():
    run(["4", "emulate"])


def test_eight_ranks_emulated_on_one_gpu():
    run(["8", "emulate"])


@pytest.mark.multigpu
def test_one_gpu_per_rank():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    run([str(min(n, 8))])
