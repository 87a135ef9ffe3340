import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


# Run order: in-process kernel tests first, then the files that start child processes on the GPU or
# work on page-locked host memory, then the allocation-free entry point (its file must come last).
_LATE = ("test_multigpu.py", "test_cpp_harness_gpu.py", "test_zero_copy_io_gpu.py", "test_checked_build_gpu.py",
         "test_zz_no_alloc.py")


def pytest_collection_modifyitems(config, items):
    import torch

    def rank(item):
        name = os.path.basename(str(getattr(item, "path", None) or item.fspath))
        return _LATE.index(name) + 1 if name in _LATE else 0

    items.sort(key=rank)

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
