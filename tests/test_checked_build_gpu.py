"""The range-checking flavour of the library (`_C_bounds.so`, TDX_BOUNDS=1).

It stands in for a memory checker on the peer-mapped stores: every store of the fused all-reduce
kernels into a symmetric allocation is compared with the allocation's extent first. The child
process checks that correct runs stay clean under the checks, and that a store which leaves a
(deliberately shortened) extent is recorded as status 7 and redirected to a scratch slot - nothing
is written out of range, nothing faults, and the kernel leaves through its bounded wait."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_checked_flavour_runs_clean_and_catches_a_short_extent():
    lib = os.path.join(os.path.dirname(HERE), "torch_dist_ext_b200", "_C_bounds.so")
    assert os.path.exists(lib), "build the checked flavour: python -m torch_dist_ext_b200._build --bounds"
    env = dict(os.environ, TDX_BOUNDS="1")
    out = subprocess.run([sys.executable, os.path.join(HERE, "checked_build_worker.py")], env=env,
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "checked build ok" in out.stdout
