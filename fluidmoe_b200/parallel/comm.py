"""All-to-all primitives on ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

These are the *baseline* transports: the same data movement the fused kernels perform from
inside GEMM epilogues is done here with library collectives, which is what the reference does in
its backward pass and what the correctness tests compare against.

Counterpart of fluid/core/comm.py:35-258 of the reference.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist


class SplitMismatchError(RuntimeError):
    """The split sizes passed by the ranks of a group do not describe one consistent exchange."""


def group_size(group) -> int:
    if group is None:
        return dist.get_world_size() if dist.is_initialized() else 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None:
        return dist.get_rank() if dist.is_initialized() else 0
    return dist.get_rank(group)


def check_split_matrix(input_splits: Optional[List[int]], output_splits: Optional[List[int]],
                       group, numel_dim0: int) -> None:
    """Gather every rank's split lists and verify ``send[src][dst] == recv[dst][src]``.

    Enabled by ``FLUID_DEBUG_A2A_SPLITS=1`` (costs a host-side all-gather per call).
    """
    world = group_size(group)
    me = (list(input_splits) if input_splits is not None else [numel_dim0 // world] * world,
          list(output_splits) if output_splits is not None else None)
    gathered = [None] * world
    dist.all_gather_object(gathered, me, group=group)
    for src in range(world):
        for dst in range(world):
            sent = gathered[src][0][dst]
            recv_list = gathered[dst][1]
            if recv_list is None:
                continue
            if recv_list[src] != sent:
                raise SplitMismatchError(
                    f"all-to-all split mismatch: rank {src} sends {sent} rows to rank {dst}, "
                    f"which expects {recv_list[src]}")


def _debug_check_alltoallv_splits(input_rows: int, output_rows: int, input_split_sizes: Optional[List[int]],
                                  output_split_sizes: Optional[List[int]], group, tag: str = "") -> None:
    """Checks of an all-to-all-v call under the reference's name and argument order
    (fluid/core/comm.py:98-105).  Does nothing unless ``FLUID_DEBUG_A2A_SPLITS=1`` and both lists
    are given; then the lists must have one entry per rank, add up to the rows of the buffers they
    describe, and agree across ranks (``check_split_matrix``)."""
    if os.environ.get("FLUID_DEBUG_A2A_SPLITS", "0") != "1":
        return
    if input_split_sizes is None or output_split_sizes is None:
        return
    world, me = group_size(group), group_rank(group)
    ins, outs = [int(v) for v in input_split_sizes], [int(v) for v in output_split_sizes]
    where = f"all-to-all-v '{tag}' on rank {me}"
    if len(ins) != world or len(outs) != world:
        raise SplitMismatchError(f"{where}: {len(ins)} input and {len(outs)} output splits for {world} ranks")
    if sum(ins) != int(input_rows):
        raise SplitMismatchError(f"{where}: input splits add up to {sum(ins)}, the buffer has {input_rows} rows")
    if sum(outs) != int(output_rows):
        raise SplitMismatchError(f"{where}: output splits add up to {sum(outs)}, the buffer has {output_rows} rows")
    if world > 1:
        check_split_matrix(ins, outs, group, int(input_rows))


def all_to_all(x: torch.Tensor, group=None, input_splits: Optional[List[int]] = None,
               output_splits: Optional[List[int]] = None,
               output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exchange dim-0 slices of ``x`` between the ranks of ``group``.

    Equal splits when no lists are given, all-to-all-v otherwise.  A group of one rank returns a
    copy so that callers may always treat the result as a fresh buffer.
    """
    world = group_size(group)
    if world == 1:
        if output is not None:
            output.copy_(x)
            return output
        return x.clone()
    x = x.contiguous()
    if os.environ.get("FLUID_DEBUG_A2A_SPLITS", "0") == "1":
        check_split_matrix(input_splits, output_splits, group, x.shape[0])
    if output is None:
        rows = sum(output_splits) if output_splits is not None else x.shape[0]
        output = torch.empty((rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        # The collective may run on a side stream: keep both buffers alive for that stream.
        stream = torch.cuda.current_stream()
        x.record_stream(stream)
        output.record_stream(stream)
    dist.all_to_all_single(output, x, output_split_sizes=output_splits,
                           input_split_sizes=input_splits, group=group)
    return output


_all_to_all = all_to_all


def sp2hp(x: torch.Tensor, group=None, output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sequence-parallel -> head-parallel: ``[s/P, b, H, d] -> [s, b, H/P, d]``.

    Rank p receives head block p of every rank's sequence block; sequence blocks are concatenated
    in rank order.
    """
    P = group_size(group)
    if P == 1:
        return x if output is None else output.copy_(x)
    s_loc, b, H, d = x.shape
    assert H % P == 0, (H, P)
    send = x.view(s_loc, b, P, H // P, d).permute(2, 0, 1, 3, 4).contiguous()
    out = output if output is not None else torch.empty(
        P * s_loc, b, H // P, d, dtype=x.dtype, device=x.device)
    all_to_all(send.view(P * s_loc, b, H // P, d), group, output=out.view(P * s_loc, b, H // P, d))
    return out


def hp2sp(x: torch.Tensor, group=None, output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Head-parallel -> sequence-parallel: ``[s, b, H/P, d] -> [s/P, b, H, d]``."""
    P = group_size(group)
    if P == 1:
        return x if output is None else output.copy_(x)
    s, b, h_loc, d = x.shape
    assert s % P == 0, (s, P)
    s_loc = s // P
    raw = all_to_all(x.contiguous(), group)  # [P * s_loc, b, h_loc, d], block p from rank p
    res = raw.view(P, s_loc, b, h_loc, d).permute(1, 2, 0, 3, 4)
    if output is not None:
        output.view(s_loc, b, P, h_loc, d).copy_(res)
        return output
    return res.contiguous().view(s_loc, b, P * h_loc, d)


_all_to_all_sp2hp_forward = sp2hp
_all_to_all_hp2sp_forward = hp2sp
