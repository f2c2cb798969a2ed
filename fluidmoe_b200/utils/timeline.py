"""Arithmetic on a device timeline: lists of ``(start, end, name)`` kernel records in one time unit.

Used by the step profile of ``bench.py`` to answer two questions the reference answers with an
external timeline viewer (``tests/nsys_fluidmoe.py:52-160`` drives the capture, the reading is
manual): where did the device sit idle, and which compute kernels ran while a collective kernel
held SMs on another stream.
"""
from __future__ import annotations

from typing import Iterable, List, Sequence, Tuple

Interval = Tuple[float, float]
Record = Tuple[float, float, str]


def merge_intervals(intervals: Iterable[Interval]) -> List[Interval]:
    """Union of intervals as a sorted list of disjoint intervals (touching ones are joined)."""
    out: List[Interval] = []
    for st, en in sorted((s, e) for s, e in intervals if e > s):
        if out and st <= out[-1][1]:
            if en > out[-1][1]:
                out[-1] = (out[-1][0], en)
        else:
            out.append((st, en))
    return out


def overlap(start: float, end: float, merged: Sequence[Interval]) -> float:
    """Length of ``[start, end]`` covered by ``merged`` (disjoint intervals, e.g. from merge_intervals)."""
    return sum(max(0.0, min(end, en) - max(start, st)) for st, en in merged)


def idle_gaps(records: Iterable[Record]):
    """``(span, idle, gaps)`` of a timeline: time from the first start to the last end, the part of
    it during which no kernel ran, and every gap as ``(length, name before, name after)`` in time
    order.  Kernels on different streams may overlap; a gap is time that no stream filled."""
    recs = sorted(records)
    if not recs:
        return 0.0, 0.0, []
    gaps, idle = [], 0.0
    busy_end, prev = recs[0][1], recs[0][2]
    for st, en, name in recs[1:]:
        if st > busy_end:
            gaps.append((st - busy_end, prev, name))
            idle += st - busy_end
        if en > busy_end:
            busy_end, prev = en, name
    return busy_end - recs[0][0], idle, gaps
