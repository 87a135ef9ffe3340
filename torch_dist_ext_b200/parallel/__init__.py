"""Process-level plumbing: peer-buffer registration and tensor-parallel layers."""
from .comm import CommProcess, setup_env, get_comm, teardown_env, local_workspaces  # noqa: F401
