"""Wall-clock accounting of host-side orchestration (``FLUID_OVERHEAD_PROFILE=1``).

Tags are grouped into buckets by prefix: ``overhead.fwd*`` (forward overlap bookkeeping),
``overhead.bwd*`` (backward scheduling), ``overhead.ar*`` (all-reduce bookkeeping), other.
Counterpart of fluid/core/overhead_profiler.py:23-173 of the reference.
"""
from __future__ import annotations

import os
import threading
import time
from typing import Dict, Optional, Tuple


class OverheadProfiler:
    BUCKETS = (("overhead.fwd", "fwd_tournament"), ("overhead.bwd", "bwd_refinement"),
               ("overhead.ar", "ar_bookkeeping"))

    def __init__(self, enabled: Optional[bool] = None):
        self.enabled = (os.environ.get("FLUID_OVERHEAD_PROFILE", "0") == "1") if enabled is None else enabled
        self._stats: Dict[str, list] = {}
        self._lock = threading.Lock()

    def set_enabled(self, enabled: bool) -> None:
        self.enabled = bool(enabled)

    def enter(self, tag: str) -> Optional[Tuple[str, float]]:
        return (tag, time.perf_counter()) if self.enabled else None

    def exit(self, token) -> None:
        if token is None:
            return
        tag, t0 = token
        dt = (time.perf_counter() - t0) * 1e3
        with self._lock:
            st = self._stats.setdefault(tag, [0.0, 0])
            st[0] += dt
            st[1] += 1

    def measure(self, tag: str):
        prof = self

        class _Ctx:
            def __enter__(self_inner):
                self_inner.tok = prof.enter(tag)

            def __exit__(self_inner, *exc):
                prof.exit(self_inner.tok)
                return False
        return _Ctx()

    def reset(self) -> None:
        with self._lock:
            self._stats.clear()

    def get_stats(self) -> Dict[str, Dict[str, float]]:
        with self._lock:
            return {k: {"total_ms": v[0], "count": v[1]} for k, v in self._stats.items()}

    def summary_by_bucket(self, num_iters: int = 1) -> Dict[str, float]:
        n = max(1, num_iters)
        out = {name: 0.0 for _, name in self.BUCKETS}
        out["other"] = 0.0
        for tag, st in self.get_stats().items():
            for prefix, name in self.BUCKETS:
                if tag.startswith(prefix):
                    out[name] += st["total_ms"] / n
                    break
            else:
                out["other"] += st["total_ms"] / n
        out["total"] = sum(out.values())
        return out


_PROFILER = OverheadProfiler()


def get_overhead_profiler() -> OverheadProfiler:
    return _PROFILER


# module-level conveniences mirroring the function-style API
def set_enabled(enabled: bool) -> None:
    _PROFILER.set_enabled(enabled)


def enter(tag: str):
    return _PROFILER.enter(tag)


def exit(token) -> None:  # noqa: A001 - name kept for API compatibility
    _PROFILER.exit(token)


def measure(tag: str):
    return _PROFILER.measure(tag)


def reset() -> None:
    _PROFILER.reset()


def get_stats():
    return _PROFILER.get_stats()


def summary_by_bucket(num_iters: int = 1):
    return _PROFILER.summary_by_bucket(num_iters)
