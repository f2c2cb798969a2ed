"""Process groups and per-process parallel context.

Ranks are laid out as ``[dp][cp]`` with ``ep == cp`` (the constraint every driver of the reference
enforces, tests/run_block_benchmark.py:280): consecutive ranks form one sequence-/expert-parallel
group; ranks with the same position in their group form an expert-data-parallel group; the whole
world is the dense data-parallel group (dense parameters are replicated over dp x cp).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelContext:
    world_size: int = 1
    rank: int = 0
    cp_size: int = 1
    ep_size: int = 1
    dp_size: int = 1
    cp_group: Optional[object] = None
    ep_group: Optional[object] = None
    dp_cp_group: Optional[object] = None      # dense-parameter gradient group (whole world)
    expert_dp_group: Optional[object] = None  # ranks holding the same experts
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    fused_ctx: Optional[object] = None

    @property
    def cp_rank(self) -> int:
        return dist.get_rank(self.cp_group) if (self.cp_group is not None and dist.is_initialized()) else 0


def init_distributed(backend: Optional[str] = None, device: Optional[torch.device] = None) -> torch.device:
    """Initialise ``torch.distributed`` from the torchrun environment (no-op for one process)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if device is None:
        if torch.cuda.is_available():
            torch.cuda.set_device(local_rank)
            device = torch.device("cuda", local_rank)
        else:
            device = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        backend = backend or ("nccl" if device.type == "cuda" else "gloo")
        kw = {}
        if device.type == "cuda":
            kw["device_id"] = device
        dist.init_process_group(backend=backend, **kw)
    return device


def init_parallel(ep_size: Optional[int] = None, cp_size: Optional[int] = None, device=None,
                  symmetric_heap_bytes: int = 0) -> ParallelContext:
    """Build the parallel context.  ``ep_size`` defaults to the world size; ``cp_size`` to ``ep_size``.

    With ``symmetric_heap_bytes > 0`` on GPUs a symmetric heap over the expert-parallel group is
    created and the fused (device-initiated) communication paths become available."""
    if not dist.is_initialized():
        dev = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        return ParallelContext(device=dev)
    world, rank = dist.get_world_size(), dist.get_rank()
    ep = ep_size or world
    cp = cp_size or ep
    assert ep == cp, "expert-parallel and sequence-parallel sizes must be equal"
    assert world % cp == 0
    dp = world // cp
    dev = torch.device(device) if device is not None else (
        torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    cp_group = ep_group = None
    for d in range(dp):
        ranks = list(range(d * cp, (d + 1) * cp))
        g = dist.new_group(ranks)
        if rank in ranks:
            cp_group = ep_group = g
    expert_dp_group = None
    for c in range(cp):
        ranks = list(range(c, world, cp))
        g = dist.new_group(ranks)
        if rank in ranks:
            expert_dp_group = g
    ctx = ParallelContext(world, rank, cp, ep, dp, cp_group, ep_group, dist.group.WORLD, expert_dp_group, dev)
    if symmetric_heap_bytes > 0 and dev.type == "cuda" and cp > 1:
        from .parallel.fused import FusedCommContext
        ctx.fused_ctx = FusedCommContext(ep_group, symmetric_heap_bytes, dev)
    return ctx
