"""Peer-buffer registration across ranks.

Counterpart of the reference's ``CommProcess`` and ``setup_env``
(torch_dist_ext/__init__.py:19-46): every rank allocates one symmetric workspace, the opaque
handles are exchanged ONCE with ``all_gather_object`` over whatever process group the caller
initialised, every rank maps every peer, and two barriers bracket the mapping. Differences:
the CUDA device is ``torch.cuda.current_device()`` unless given (the reference forces
``device == rank``); a CPU-only process group (gloo) gets a pure-PyTorch communicator with the
same interface so that the plumbing is testable without GPUs; ``teardown_env`` exists.
"""
from __future__ import annotations

import atexit
import logging
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..utils.config import ALGO_NAMES, config

log = logging.getLogger("torch_dist_ext_b200")

DEFAULT_MAX_BYTES = 8192 * 16384  # 128 MiB, the reference's default (torch_dist_ext/__init__.py:41)
NBLOCKS = 256                     # kept for constructor parity with the reference


class CommProcess:
    """Owns this rank's workspace and its registration with the peers."""

    def __init__(self, rank: int, world_size: int, size_in_bytes: int = DEFAULT_MAX_BYTES,
                 group: Optional[dist.ProcessGroup] = None, device: Optional[int] = None):
        self.rank, self.world_size, self.group = rank, world_size, group
        self.size_in_bytes = size_in_bytes
        self.is_cuda = torch.cuda.is_available()
        self.algo_counts = {}
        self.lamport_bytes = config.lamport_mb << 20
        if not self.is_cuda:
            # CPU ranks (gloo): no device buffers; the op runs the PyTorch statement of itself.
            self.comm = None
            self.device = torch.device("cpu")
            self._exchange_cpu()
            return
        if device is None:
            # Same convention as the reference when the caller has not chosen a device yet.
            if world_size > 1 and torch.cuda.device_count() >= world_size and torch.cuda.current_device() == 0:
                device = rank
            else:
                device = torch.cuda.current_device()
        torch.cuda.set_device(device)
        self.device = torch.device("cuda", device)
        self.comm = _lib.ops().create_workspace(rank, world_size, NBLOCKS, size_in_bytes, config.lamport_mb << 20,
                                                device, 1 if (config.nvls and world_size > 1) else 0)
        self.comm.set_timeout_ms(config.timeout_ms)
        if world_size > 1:
            handle = self.comm.get_handle()
            handle_list: List[Optional[torch.Tensor]] = [None] * world_size
            dist.all_gather_object(handle_list, handle, group=group)
            torch.cuda.synchronize(device)
            dist.barrier(group=group)
            self.comm.open_handles(handle_list)
            torch.cuda.synchronize(device)
            # NVLS is used only if EVERY rank joined the multicast object
            flags: List[Optional[bool]] = [None] * world_size
            dist.all_gather_object(flags, bool(self.comm.has_multicast()), group=group)
            if not all(flags) and self.comm.has_multicast():
                self.comm.disable_multicast()
            if not all(flags):
                log.info("NVLS disabled: %s", self.comm.multicast_note() or "a peer could not join the multicast object")
            dist.barrier(group=group)
        for n, entry in config.policy.items():
            _lib.ops().set_policy(n, *entry)
        self._table = self.comm.get_workspace(torch.empty(0, device=self.device))

    def _exchange_cpu(self) -> None:
        if self.world_size > 1:
            ids: List[Optional[int]] = [None] * self.world_size
            dist.all_gather_object(ids, self.rank, group=self.group)
            if ids != list(range(self.world_size)):
                raise RuntimeError(f"rank order mismatch during registration: {ids}")
            dist.barrier(group=self.group)

    def get_workspace(self, ref: torch.Tensor) -> torch.Tensor:
        if self.comm is None:
            return torch.zeros(table_nbytes(), dtype=torch.uint8)
        return self._table

    def get_workspace_copy(self, ref: torch.Tensor) -> torch.Tensor:
        """A fresh tensor with the table's contents that the ops accept like the table itself."""
        if self.comm is None:
            return torch.zeros(table_nbytes(), dtype=torch.uint8)
        copy = self._table.clone()
        self.comm.adopt_table(copy)
        return copy

    def reset(self) -> None:
        """Collective re-initialisation of flags, epochs and sentinels."""
        if self.comm is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world_size > 1:
            dist.barrier(group=self.group)
        self.comm.reset()
        if self.world_size > 1:
            dist.barrier(group=self.group)

    def check(self) -> None:
        """Raise if a device-side wait ran out since the last reset (non-blocking read)."""
        if self.comm is not None and self.comm.errors_seen() != 0:
            s = self.stats()
            raise RuntimeError(
                "torch_dist_ext_b200: a device-side wait timed out: "
                f"code={s['status'][0]} rank={s['status'][1]} peer={s['status'][2]} phase={s['status'][3]} "
                f"block={s['status'][4]} row={s['status'][5]} (errors={s['error_count']}). "
                "Outputs of that call are invalid; call reset() on all ranks before reuse.")

    def stats(self) -> dict:
        if self.comm is None:
            return {"backend": "cpu", "algo_counts": dict(self.algo_counts)}
        v = self.comm.stats()
        return {
            "backend": "cuda", "total_bytes": v[0], "lamport_bytes": v[1], "stage_bytes": v[2],
            "error_count": v[3], "lamport_epoch": v[4], "barrier_epoch": v[5], "has_multicast": bool(v[6]),
            "status": v[7:15], "algo_counts": {ALGO_NAMES.get(k, k): n for k, n in self.algo_counts.items()},
        }


def table_nbytes() -> int:
    """Size of the tensor returned by ``get_workspace`` (the device-resident pointer table)."""
    return int(_lib.ops().table_nbytes())


_comm: Optional[CommProcess] = None
_world_size: Optional[int] = None


def setup_env(rank: int, world_size: int, max_size_in_bytes: int = DEFAULT_MAX_BYTES,
              group: Optional[dist.ProcessGroup] = None, device: Optional[int] = None) -> CommProcess:
    """Allocate and register this rank's workspace (once per process)."""
    global _comm, _world_size
    if world_size > 1 and not dist.is_initialized():
        raise RuntimeError("setup_env needs an initialised torch.distributed process group")
    _comm = CommProcess(rank, world_size, max_size_in_bytes, group, device)
    _world_size = world_size
    return _comm


def teardown_env() -> None:
    """Collective: wait for the device, agree with the peers that nobody is still using the
    buffers, then unmap and free them (multicast bindings included)."""
    global _comm, _world_size
    if _comm is not None and _comm.is_cuda:
        torch.cuda.synchronize(_comm.device)
        if _comm.world_size > 1 and dist.is_initialized():
            try:
                dist.barrier(group=_comm.group)
            except Exception:  # the group may already be gone at interpreter exit
                pass
        _comm.comm = None
        _comm._table = None
    _comm = None
    _world_size = None


atexit.register(teardown_env)


def get_comm() -> CommProcess:
    if _comm is None:
        raise RuntimeError("call setup_env(rank, world_size) first")
    return _comm


def world_size() -> Optional[int]:
    return _world_size


def local_workspaces(world_size: int, size_in_bytes: int = 16 << 20, timeout_ms: Optional[int] = None):
    """``world_size`` workspaces on the CURRENT device, registered with each other inside this
    process. For the single-GPU emulation of the multi-rank kernels."""
    # multicast off: every emulated rank lives on the same device, which can join a multicast
    # object only once
    ws = [_lib.ops().create_workspace(r, world_size, NBLOCKS, size_in_bytes, 0, -1, 0) for r in range(world_size)]
    if world_size > 1:
        _lib.ops().connect_local(ws)
    for w in ws:
        w.set_timeout_ms(config.timeout_ms if timeout_ms is None else timeout_ms)
    return ws
