"""The descriptor channel of the workspace manager (csrc/fd_channel.cpp), across two processes.

Host-only C++: compiled here with g++ and run as a program, so it needs neither a GPU nor the
built extension."""
import os
import shutil
import subprocess

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_descriptor_travels_between_processes(tmp_path):
    exe = tmp_path / "fd_channel_test"
    subprocess.run(["g++", "-std=c++17", "-pthread", "-I", os.path.join(REPO, "torch_dist_ext_b200", "csrc", "include"),
                    os.path.join(REPO, "tests", "cpp", "fd_channel_test.cpp"),
                    os.path.join(REPO, "torch_dist_ext_b200", "csrc", "fd_channel.cpp"), "-o", str(exe)],
                   check=True, timeout=120)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    assert "ok" in out.stdout
