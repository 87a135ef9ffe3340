"""Drop-in name for code written against the reference package: ``import torch_dist_ext`` gives
the same ``setup_env`` / ``get_workspace`` / ``allreduce_rms`` / ``CommProcess`` / ``CommWorkspace``
names (reference: torch_dist_ext/__init__.py:15-84), backed by torch_dist_ext_b200."""
from torch_dist_ext_b200 import *  # noqa: F401,F403
from torch_dist_ext_b200 import (CommProcess, CommWorkspace, allreduce_rms, allreduce_rms_fusion_impl,  # noqa: F401
                                 get_workspace, setup_env)


def __getattr__(name):
    # the reference keeps its registration state in two module globals (torch_dist_ext/__init__.py:37-38)
    from torch_dist_ext_b200.parallel import comm as _c

    if name == "comm":
        return _c._comm
    if name == "world_size_":
        return _c.world_size()
    raise AttributeError(f"module 'torch_dist_ext' has no attribute {name!r}")
