"""Host-side liveness checks between training steps.

The reference has no failure handling: a worker thread that dies leaves every poll hanging
(ref hp_cuda.cpp:805-809).  Here the device side reports through status words (bounded flag
waits, payload bounds checks) and the host side through this heartbeat: every rank publishes
the step it has finished to a ``torch.distributed`` store; before launching the next step a
rank checks that all peers have reached the same step and otherwise learns *which* peers
are gone -- on the host, with nothing in flight on the GPU -- so that it can stop, shrink the
job or restore from a checkpoint instead of waiting for a flag that will never come.
"""
from __future__ import annotations

import time
from typing import List


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "hipress/hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int) -> None:
        """Publish that this rank has finished ``step``."""
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self) -> None:
        """Announce an orderly departure (between steps, nothing in flight)."""
        self.store.set(self._key(self.rank), "left")

    def peer_step(self, rank: int):
        """Latest step of ``rank``; -1 if it never reported, None if it left."""
        try:
            if not self.store.check([self._key(rank)]):
                return -1
            v = self.store.get(self._key(rank)).decode()
        except Exception:
            return -1
        return None if v == "left" else int(v)

    def missing(self, step: int, timeout_s: float = 5.0, poll_s: float = 0.01) -> List[int]:
        """Ranks that have not finished ``step`` within ``timeout_s`` (or that left)."""
        deadline = time.monotonic() + timeout_s
        pending = [r for r in range(self.world) if r != self.rank]
        gone: List[int] = []
        while pending:
            still = []
            for r in pending:
                s = self.peer_step(r)
                if s is None:
                    gone.append(r)
                elif s < step:
                    still.append(r)
            pending = still
            if not pending or time.monotonic() > deadline:
                break
            time.sleep(poll_s)
        return sorted(gone + pending)
