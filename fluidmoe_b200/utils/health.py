"""Host-side health checks: a heartbeat through the rendezvous store and a status-word poll.

Ranks call ``beat()`` between steps; ``missing()`` lists ranks whose last beat is older than
``stale_after_s``.  Together with the kernels' bounded waits (which turn a peer that never signals
into a ``FluidKernelTimeout`` on the host) this is the failure-detection layer: nothing here can
hang or fault a GPU.  The reference has no failure detection of its own.
"""
from __future__ import annotations

import time
from typing import List


class Heartbeat:
    def __init__(self, store, rank: int, world: int, stale_after_s: float = 30.0, prefix: str = "fm_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.stale_after_s = stale_after_s
        self.prefix = prefix

    def beat(self) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", repr(time.time()))

    def missing(self) -> List[int]:
        now = time.time()
        out = []
        for r in range(self.world):
            try:
                last = float(self.store.get(f"{self.prefix}/{r}").decode())
            except Exception:  # noqa: BLE001 - never written
                out.append(r)
                continue
            if now - last > self.stale_after_s:
                out.append(r)
        return out


def check_kernels() -> None:
    """Raise ``FluidKernelTimeout`` if any kernel recorded a bounded-wait expiry (host sync)."""
    from ..ops.gemm import check_status
    check_status()
