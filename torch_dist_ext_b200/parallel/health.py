"""Host-side failure detection: membership and heartbeats over the process group's store.

The device side already bounds every wait (a kernel whose peer never arrives returns with an error
record instead of hanging). This module is the other half: ranks learn ON THE HOST that a peer has
left or stopped, BEFORE they launch a kernel that would store into that peer's memory. A rank that
leaves announces it (``leave()``); a rank that stops without announcing is caught by its heartbeat
age. ``check()`` is cheap enough to call before every step of a serving loop.

The reference has no failure handling (its four device-side spins are unbounded,
src/common/all_reduce_fusion_impl.h:81, :118, :189, :456).
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch.distributed as dist


class PeerLeft(RuntimeError):
    """A peer announced that it left, or its heartbeat is older than the allowed age."""


class Membership:
    def __init__(self, rank: int, world_size: int, store: Optional["dist.Store"] = None, prefix: str = "tdx/health",
                 max_age_s: float = 10.0):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.rank, self.world, self.store, self.prefix, self.max_age = rank, world_size, store, prefix, max_age_s
        self.beat()

    def _key(self, kind: str, r: int) -> str:
        return f"{self.prefix}/{kind}/{r}"

    def beat(self) -> None:
        """Record that this rank is alive now."""
        self.store.set(self._key("beat", self.rank), repr(time.time()))

    def leave(self, reason: str = "") -> None:
        """Announce an orderly departure (call between steps, with no kernel or collective in flight)."""
        self.store.set(self._key("left", self.rank), reason or "left")

    def departed(self) -> List[int]:
        out = []
        for r in range(self.world):
            if r != self.rank and self.store.check([self._key("left", r)]):
                out.append(r)
        return out

    def stale(self) -> List[int]:
        now, out = time.time(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            if not self.store.check([self._key("beat", r)]):
                out.append(r)
                continue
            if now - float(self.store.get(self._key("beat", r)).decode()) > self.max_age:
                out.append(r)
        return out

    def check(self, heartbeats: bool = True) -> None:
        """Raise PeerLeft if a peer left or went silent; otherwise refresh this rank's heartbeat."""
        gone = self.departed()
        if gone:
            raise PeerLeft(f"rank(s) {gone} left the job; do not launch collectives that touch their memory")
        if heartbeats:
            silent = self.stale()
            if silent:
                raise PeerLeft(f"rank(s) {silent} have not reported for more than {self.max_age} s")
        self.beat()
