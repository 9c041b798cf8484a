"""Host-side peer liveness for an EP group.

The device barriers of this library are bounded (a peer that never arrives costs one timeout and
an exception, not a hang), but the cheaper place to learn that a rank has gone is the host,
BEFORE the next kernel is launched.  ``Heartbeat`` keeps one counter per rank in the process
group's key-value store: a rank publishes the step it is about to run, and waits (with a short
limit) until every peer has published it too.  A rank that left between steps therefore turns
into a ``PeerLostError`` on the others with no kernel or collective in flight.
The reference has no failure handling beyond a 100 s spin and a trap (moonep/_common.py:36,335-341).
"""
from __future__ import annotations

import time
from typing import Optional

import torch.distributed as dist


class PeerLostError(RuntimeError):
    def __init__(self, missing, step):
        self.missing, self.step = list(missing), step
        super().__init__(f"ranks {self.missing} did not reach step {step}")


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, prefix: str = "moonep_b200/hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.prefix = prefix

    @classmethod
    def from_default_group(cls, prefix: str = "moonep_b200/hb") -> "Heartbeat":
        store = dist.distributed_c10d._get_default_store()
        return cls(store, dist.get_rank(), dist.get_world_size(), prefix)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        """Publish that this rank is about to run ``step``."""
        self.store.set(self._key(self.rank), str(step))

    def _peer_step(self, r: int) -> int:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return -1
            return int(self.store.get(self._key(r)).decode())
        except Exception:  # noqa: BLE001 - a store error counts as "not seen"
            return -1

    def wait_for_peers(self, step: int, timeout_s: float = 5.0, poll_s: float = 0.01) -> None:
        """Return when every rank has published ``>= step``; raise ``PeerLostError`` otherwise."""
        deadline = time.monotonic() + timeout_s
        missing = [r for r in range(self.world) if r != self.rank]
        while True:
            missing = [r for r in missing if self._peer_step(r) < step]
            if not missing:
                return
            if time.monotonic() > deadline:
                raise PeerLostError(missing, step)
            time.sleep(poll_s)

    def step(self, step: int, timeout_s: float = 5.0) -> None:
        """``beat`` then ``wait_for_peers``: call at the top of every training step."""
        self.beat(step)
        self.wait_for_peers(step, timeout_s)
