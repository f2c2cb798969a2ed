"""Round-robin tournament order and the per-layer overlap context.

On NVSwitch every peer is reachable at full bandwidth, so the tournament is not needed to spread
load over links; it is kept as the *consumption order* of peer data (local block first, then
partners in round order), for the NCCL / gloo point-to-point path, and for API compatibility.

Counterpart of fluid/core/comm.py:265-392 of the reference.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .streams import get_stream_manager


def compute_round_robin_schedule(num_ranks: int) -> List[List[Tuple[int, int]]]:
    """Circle-method tournament: ``schedule[round] = [(a, b), ...]`` with ``a < b``.

    An even number of ranks P needs P-1 rounds and every rank plays in each; an odd number needs P
    rounds and one rank idles per round (it is paired with a phantom player).  Seat 0 is fixed and
    the other seats rotate by one per round; seat i meets seat n-1-i.
    """
    if num_ranks <= 1:
        return []
    n = num_ranks + (num_ranks & 1)  # players including the phantom
    ring = n - 1

    def player_at(seat: int, rnd: int) -> int:
        return 0 if seat == 0 else 1 + (seat - 1 - rnd) % ring

    schedule = []
    for rnd in range(ring):
        pairs = []
        for seat in range(n // 2):
            a, b = player_at(seat, rnd), player_at(n - 1 - seat, rnd)
            if a >= num_ranks or b >= num_ranks:
                continue  # phantom: the real player idles
            pairs.append((min(a, b), max(a, b)))
        schedule.append(pairs)
    return schedule


def partner_table(num_ranks: int) -> List[List[int]]:
    """``table[rank][round]`` = partner of ``rank`` in ``round`` (-1 when idle)."""
    sched = compute_round_robin_schedule(num_ranks)
    table = [[-1] * len(sched) for _ in range(num_ranks)]
    for rnd, pairs in enumerate(sched):
        for a, b in pairs:
            table[a][rnd] = b
            table[b][rnd] = a
    return table


class MultiCardOverlapContext:
    """Resources shared by the overlap paths of one layer: schedule, side stream, named events."""

    def __init__(self, device, ep_size: int, cp_size: Optional[int] = None):
        self.device = torch.device(device)
        self.ep_size = ep_size
        self.cp_size = cp_size if cp_size is not None else ep_size
        self.schedule = compute_round_robin_schedule(ep_size)
        self.num_rounds = len(self.schedule)
        self._partners = partner_table(ep_size)
        self._sm = get_stream_manager(self.device)
        self._sm.initialize(self.device)
        self._cache: Dict[Tuple[int, int], int] = {}

    @property
    def comm_stream(self):
        return self._sm.comm_stream

    @property
    def data_ready_event(self):
        return self._sm.data_ready_event

    def get_stream(self):
        return self.comm_stream

    def get_partner(self, my_rank: int, round_idx: int) -> int:
        if my_rank >= len(self._partners) or round_idx >= self.num_rounds or round_idx < 0:
            return -1
        return self._partners[my_rank][round_idx]

    def partners_in_order(self, my_rank: int) -> List[int]:
        """Partners of ``my_rank`` in round order, idle rounds skipped."""
        return [p for p in self._partners[my_rank] if p >= 0] if self.ep_size > 1 else []

    def get_round_event(self, tag: str, round_idx: int):
        return self._sm.get_sync_event(("overlap", tag, round_idx))
