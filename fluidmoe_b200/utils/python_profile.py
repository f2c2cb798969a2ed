"""Named wall-clock sections for Python-side code (``FLUID_PROFILE_PYTHON=1``).

Counterpart of fluid/core/python_profile.py:7-44 of the reference.
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Dict

ENABLED = os.environ.get("FLUID_PROFILE_PYTHON", "0") == "1"
_STATS: Dict[str, Dict[str, float]] = {}


@contextlib.contextmanager
def profile_section(name: str):
    if not ENABLED:
        yield
        return
    t0 = time.perf_counter()
    try:
        yield
    finally:
        st = _STATS.setdefault(name, {"total_ms": 0.0, "count": 0})
        st["total_ms"] += (time.perf_counter() - t0) * 1e3
        st["count"] += 1


def reset_profile_stats() -> None:
    _STATS.clear()


def get_profile_stats() -> Dict[str, Dict[str, float]]:
    return {k: dict(v) for k, v in _STATS.items()}
