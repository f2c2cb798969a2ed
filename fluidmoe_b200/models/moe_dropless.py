"""Dropless expert-parallel MoE: every routed (token, expert) pair is kept, so the exchanges use
variable split sizes (all-to-all-v) and the experts run as a grouped GEMM over row groups whose
sizes are only known on the device.

The reference routes with a fixed padded capacity and drops tokens under imbalance
(fluid/moe/forward.py:387-417); its README-era API carried ``input_splits / output_splits``
(README:62-67).  This module is the variable-split path of the layer (``capacity_factor <= 0``):

* sender side: pairs sorted by expert (stable in token order); ``slot_of_token[t, j]`` is the slot of
  the j-th choice of token t, used by the same gather-sum un-permute as the padded path;
* exchange: split sizes come from the per-expert counts (one small host read per layer and
  direction; the fused device-initiated path does not apply here yet);
* receiver side: rows are placed expert-major with every expert's run padded to a multiple of 128
  rows of zeros, so that the weight-gradient GEMM can contract in whole 64-row blocks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import gemm, permute
from ..parallel import comm

_ALIGN = 128


@dataclass
class DroplessPlan:
    sorted_indices: torch.Tensor     # [T*k] token of every slot, expert-major
    permuted_probs: torch.Tensor     # [T*k] fp32
    slot_of_token: torch.Tensor      # [T, k] int32
    counts: torch.Tensor             # [E] int32 routed pairs per expert (this rank's tokens)
    input_splits: List[int]          # rows sent to every EP rank
    output_splits: List[int]         # rows received from every EP rank
    group_rows: torch.Tensor         # [nle] int32 rows per local expert (all sources)
    group_offs: torch.Tensor         # [nle] int32 aligned start row of every local expert
    rows_em: int                     # rows of the expert-major buffer (padded)
    recv_to_em: torch.Tensor         # [sum(output_splits)] int64: expert-major row of every received row
    routed_per_expert: torch.Tensor  # alias of counts (API symmetry with the padded plan)


def build_plan(top_idx: torch.Tensor, top_probs: torch.Tensor, num_experts: int, ep_group) -> DroplessPlan:
    T, k = top_idx.shape
    E = num_experts
    dev = top_idx.device
    P = comm.group_size(ep_group)
    me = comm.group_rank(ep_group)
    nle = E // P
    flat_e = top_idx.reshape(-1)
    order = torch.sort(flat_e, stable=True).indices                 # pairs by expert, token order kept
    sorted_indices = (order // k).to(torch.int64)
    permuted_probs = top_probs.reshape(-1).float()[order]
    slot_of_token = torch.empty(T * k, dtype=torch.int32, device=dev)
    slot_of_token[order] = torch.arange(T * k, dtype=torch.int32, device=dev)
    counts = torch.bincount(flat_e, minlength=E).to(torch.int32)
    # counts of every rank: [P, E]
    if P > 1:
        parts = [torch.empty(E, dtype=torch.int32, device=dev) for _ in range(P)]
        dist.all_gather(parts, counts, group=ep_group)       # works on NCCL and gloo
        allc = torch.stack(parts)
    else:
        allc = counts.view(1, E)
    host = allc.cpu()                                               # the one host read
    input_splits = [int(host[me, p * nle:(p + 1) * nle].sum()) for p in range(P)]
    mine = host[:, me * nle:(me + 1) * nle].to(torch.int64)         # [P src, nle]
    output_splits = [int(mine[r].sum()) for r in range(P)]
    rows_j = mine.sum(0)                                            # rows per local expert
    padded = ((rows_j + _ALIGN - 1) // _ALIGN) * _ALIGN
    offs_j = torch.cumsum(padded, 0) - padded
    rows_em = int(padded.sum())
    # received rows arrive source-major, inside a source expert-major; place them at
    # offs[j] + (rows of expert j from earlier sources) + i
    before = torch.cumsum(mine, 0) - mine                           # [P, nle] rows of j from sources < r
    pieces = []
    for r in range(P):
        for j in range(nle):
            n = int(mine[r, j])
            if n:
                pieces.append(torch.arange(n, dtype=torch.int64) + int(offs_j[j]) + int(before[r, j]))
    recv_to_em = (torch.cat(pieces) if pieces else torch.empty(0, dtype=torch.int64)).to(dev)
    return DroplessPlan(sorted_indices, permuted_probs, slot_of_token.view(T, k), counts, input_splits,
                        output_splits, rows_j.to(torch.int32).to(dev), offs_j.to(torch.int32).to(dev),
                        rows_em, recv_to_em, counts)


def to_experts(plan: DroplessPlan, rows_permuted: torch.Tensor, ep_group) -> torch.Tensor:
    """Permuted-order rows -> expert-major buffer (zero padded)."""
    if comm.group_size(ep_group) > 1:
        recv = comm.all_to_all(rows_permuted, ep_group, plan.input_splits, plan.output_splits)
    else:
        recv = rows_permuted
    out = torch.zeros((plan.rows_em,) + tuple(rows_permuted.shape[1:]), dtype=rows_permuted.dtype,
                      device=rows_permuted.device)
    out.index_copy_(0, plan.recv_to_em, recv)
    return out


def from_experts(plan: DroplessPlan, rows_em: torch.Tensor, ep_group) -> torch.Tensor:
    """Expert-major rows -> permuted order on the token owners (the transpose of ``to_experts``)."""
    send = rows_em.index_select(0, plan.recv_to_em)
    if comm.group_size(ep_group) > 1:
        return comm.all_to_all(send, ep_group, plan.output_splits, plan.input_splits)
    return send


def forward(plan: DroplessPlan, x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, activation: str,
            ep_group, save_pre: bool = True):
    """Returns ``(combined [T*k, H] in permuted order, state for backward)``."""
    from .moe import MoEForwardState
    permuted = permute.permute_rows(x, plan.sorted_indices)
    tokens_em = to_experts(plan, permuted, ep_group)
    probs_em = to_experts(plan, plan.permuted_probs, ep_group)
    act, pre = gemm.grouped_gemm_act(tokens_em, w1, probs_em, activation=activation,
                                     group_rows=plan.group_rows, group_offs=plan.group_offs, save_pre=save_pre)
    out_em = gemm.grouped_gemm(act, w2, b_layout="kn", group_rows=plan.group_rows, group_offs=plan.group_offs)
    return from_experts(plan, out_em, ep_group), MoEForwardState(tokens_em, probs_em, pre, act)


def backward(plan: DroplessPlan, grad_combined: torch.Tensor, state, w1: torch.Tensor, w2: torch.Tensor,
             activation: str, ep_group):
    """Returns ``(dfc2_em, dpre_em, dprobs in permuted order, dperm [T*k, H])``."""
    dfc2 = to_experts(plan, grad_combined, ep_group)
    dpre, dprobs_em = gemm.grouped_gemm_dact(dfc2, w2, state.pre_em, state.probs_em, activation=activation,
                                             group_rows=plan.group_rows, group_offs=plan.group_offs)
    dprobs = from_experts(plan, dprobs_em, ep_group)
    dtok = gemm.grouped_gemm(dpre, w1, b_layout="nk", group_rows=plan.group_rows, group_offs=plan.group_offs)
    return dfc2, dpre, dprobs, from_experts(plan, dtok, ep_group)


def register_dw_tasks(plan, state, dfc2_em, dpre_em, w1_param, w2_param, layer_id: int,
                      layer_name: str, which: str = "both") -> None:
    """Queue the expert weight gradients over device-sized row groups (``plan.group_rows`` /
    ``plan.group_offs``).  ``which``: ``both``, ``w1`` or ``w2`` (the task of ``w1`` may only be
    queued after the FC1 input-gradient GEMM when its optimizer runs in the weight-gradient
    epilogue, because that epilogue overwrites ``w1``)."""
    from ..parallel.scheduler import get_backward_scheduler
    sched = get_backward_scheduler()
    nle = plan.group_rows.numel()

    def make(a, dy, param):
        def run():
            from .moe import fused_optimizer_of
            fa = fused_optimizer_of(param, sched) if sched.is_enabled() else None
            gscale = 1.0 / max(1, sched.shared_dp_world)
            if fa is not None and getattr(fa, "fused_mode", "epilogue") == "epilogue":
                fa.wgrad_update(param, a, dy, nle, grad_scale=gscale, group_rows=plan.group_rows,
                                group_offs=plan.group_offs, max_ctas=sched.dw_max_ctas)
                return None
            alpha = gscale if fa is not None else 1.0
            buf = sched._buffer_of(param) if sched.is_enabled() else None
            if buf is not None and param.main_grad.dtype == torch.float32 and a.is_cuda:
                first = not getattr(param, "_ar_buf_written", False)
                gemm.grouped_gemm_wgrad(a, dy, nle, group_rows=plan.group_rows, group_offs=plan.group_offs,
                                        out=param.main_grad, accumulate=not first, alpha=alpha,
                                        max_ctas=sched.dw_max_ctas)
                if fa is not None:
                    fa.update_on_stream(param)
                return None
            return gemm.grouped_gemm_wgrad(a, dy, nle, group_rows=plan.group_rows, group_offs=plan.group_offs,
                                           alpha=alpha)
        return run
    if which in ("both", "w2"):
        sched.register_dw_task(f"{layer_name}.w2", layer_id, make(state.act_em, dfc2_em, w2_param), w2_param)
    if which in ("both", "w1"):
        sched.register_dw_task(f"{layer_name}.w1", layer_id, make(state.tokens_em, dpre_em, w1_param), w1_param)
