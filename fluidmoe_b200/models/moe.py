"""Expert-parallel MoE block: plan, router, dispatch + FC1, FC2 + combine, and their backward.

Data layout
-----------
* *permuted* (sender side): ``[E * cap, H]`` global-expert-major; rows ``[p*S, (p+1)*S)`` with
  ``S = nle * cap`` belong to the experts of EP rank p.
* *expert-major* (receiver side): ``[nle * P * cap, H]``; the row of (local expert j, source rank
  r, slot i) is ``(j*P + r)*cap + i``, so that each local expert is one contiguous group of the
  grouped GEMM.  The reference reaches this layout only after an ``index_select`` of the
  rank-major receive buffers (fluid/moe/forward.py:959-1022); here data is *placed* there on
  arrival.

Three transports move rows between the two layouts:

``a2a``   one ``all_to_all_single`` per direction (the baseline; also what ``MoEBaseline`` uses);
``p2p``   pairwise exchanges in round-robin order on the communication stream, each overlapped
          with the expert GEMM of the block that arrived before (works on NCCL and gloo);
``fused`` device-initiated: the permute kernel stores rows straight into the destination GPU's
          expert-major buffer and raises per-row-block flags, the grouped GEMM consumes row
          blocks as their flags complete, and the FC2 epilogue stores result rows straight into
          the owner's combine buffer (symmetric memory over NVLink).

Expert output is ``FC2(act(FC1(x)) * prob)``, so un-permuting is a plain sum over the k slots of
a token (fluid/moe/forward.py:299,317).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import gemm, permute, router as router_ops
from ..parallel import comm
from ..parallel.p2p_backend import get_p2p_backend
from ..parallel.scheduler import get_backward_scheduler
from ..parallel.schedule import MultiCardOverlapContext
from ..parallel.streams import current_stream, on_stream
from ..utils.nvtx import nvtx_range
from ..utils.overhead_profiler import get_overhead_profiler

_WARNED = set()


def _warn_once(key: str, msg: str) -> None:
    if key not in _WARNED:
        _WARNED.add(key)
        if not dist.is_initialized() or dist.get_rank() == 0:
            print(f"[fluidmoe] {msg}", flush=True)


# ============================================================================================
# plan
# ============================================================================================
class EPPlan:
    """Static description of one expert-parallel exchange with fixed (padded) capacity.

    Counterpart of the reference's EPPlan (fluid/moe/forward.py:76-158).
    """

    def __init__(self, num_tokens: int, hidden_size: int, num_experts: int, top_k: int,
                 ep_group=None, capacity_factor: float = 1.0, dtype=torch.bfloat16, device=None,
                 overlap_ctx: Optional[MultiCardOverlapContext] = None):
        self.group = ep_group
        self.ep_size = comm.group_size(ep_group)
        self.ep_rank = comm.group_rank(ep_group)
        P = self.ep_size
        assert num_experts % P == 0, (num_experts, P)
        self.num_tokens, self.hidden_size = num_tokens, hidden_size
        self.num_experts, self.top_k = num_experts, top_k
        self.num_local_experts = nle = num_experts // P
        self.capacity_factor = capacity_factor
        self.expert_capacity = cap = router_ops.expert_capacity(num_tokens, top_k, num_experts, capacity_factor)
        self.S = nle * cap                      # rows exchanged with every peer
        self.rows_local = nle * P * cap         # rows of the expert-major buffer
        self.input_splits = [self.S] * P
        self.output_splits = [self.S] * P
        self.recv_total_elems = self.S * hidden_size + self.S
        self.dtype, self.device = dtype, torch.device(device) if device is not None else None
        dev = self.device
        self.expert_ids_gpu = torch.arange(num_experts, device=dev).repeat_interleave(cap)
        self.tokens_per_expert_gpu = torch.full((num_experts,), cap, dtype=torch.int32, device=dev)
        self.overlap_ctx = overlap_ctx
        self.layer_id = 0
        if overlap_ctx is not None and P > 1:
            self.partners = overlap_ctx.partners_in_order(self.ep_rank)
        else:
            self.partners = [(self.ep_rank + i) % P for i in range(1, P)]
        if ep_group is not None and dist.is_initialized():
            self.global_ranks = dist.get_process_group_ranks(ep_group)
        else:
            self.global_ranks = list(range(P))
        # per-source-rank block descriptors of the expert-major buffer (group = local expert)
        self._block_rows = torch.full((nle,), cap, dtype=torch.int32, device=dev)
        self._block_offs = [
            torch.tensor([(j * P + r) * cap for j in range(nle)], dtype=torch.int32, device=dev)
            for r in range(P)
        ]
        # where every expert-major row goes in the owner's permuted-order combine buffer
        j = torch.arange(nle, device=dev).view(nle, 1, 1)
        r = torch.arange(P, device=dev).view(1, P, 1)
        i = torch.arange(cap, device=dev).view(1, 1, cap)
        self.combine_dst_rank = r.expand(nle, P, cap).reshape(-1).to(torch.int32).contiguous()
        self.combine_dst_row = (((self.ep_rank * nle + j) * cap + i).expand(nle, P, cap)
                                .reshape(-1).to(torch.int32).contiguous())

    def block(self, src_rank: int):
        """(group_rows, group_offs) selecting the rows that came from ``src_rank``."""
        return self._block_rows, self._block_offs[src_rank]

    def dispatch_event_name(self, rnd: int) -> str:
        return f"moe_dispatch_{rnd}"

    def combine_event_name(self, rnd: int) -> str:
        return f"moe_combine_{rnd}"

    def signature(self):
        return (self.num_tokens, self.hidden_size, self.num_experts, self.top_k, self.ep_size,
                self.capacity_factor)


# ============================================================================================
# router
# ============================================================================================
def router_forward(hidden_states: torch.Tensor, router_weight: torch.Tensor, num_experts: int,
                   top_k: int, ep_group=None, capacity_factor: float = 1.0,
                   ep_plan: Optional[EPPlan] = None, router_dtype: torch.dtype = torch.float32,
                   gather_tokens: bool = True, forced_top_idx: Optional[torch.Tensor] = None,
                   logit_bias: Optional[torch.Tensor] = None):
    """Route ``hidden_states [T, H]``.

    Returns ``(permuted_tokens, permuted_probs, sorted_indices, tokens_per_expert, top_indices,
    top_probs, router_logits, routing_map, plan)`` like the reference router
    (fluid/moe/forward.py:359-466); the last element is the :class:`RoutingPlan` carrying the
    slot map used by the deterministic un-permute.  ``permuted_tokens`` is None when
    ``gather_tokens`` is False (the fused dispatch gathers rows itself).
    """
    with nvtx_range("router_forward"):
        T = hidden_states.shape[0]
        logits = router_ops.router_logits(hidden_states, router_weight, router_dtype)
        if logit_bias is not None:
            logits = logits + logit_bias.to(logits.dtype)
        top_idx, top_probs = router_ops.topk_softmax(logits, top_k, forced_top_idx)
        cap = (ep_plan.expert_capacity if ep_plan is not None
               else router_ops.expert_capacity(T, top_k, num_experts, capacity_factor))
        plan = router_ops.build_padded_plan(top_idx, top_probs, num_experts, cap)
        permuted = permute.permute_rows(hidden_states, plan.sorted_indices) if gather_tokens else None
        return (permuted, plan.permuted_probs, plan.sorted_indices, plan.tokens_per_expert, top_idx,
                top_probs, logits, plan.routing_map, plan)


# ============================================================================================
# layout helpers (rank-major <-> expert-major)
# ============================================================================================
def rank_to_expert_major(x: torch.Tensor, P: int, nle: int, cap: int) -> torch.Tensor:
    """``[P, nle, cap, ...] -> [nle, P, cap, ...]`` flattened; a view when nle == 1 or P == 1."""
    tail = x.shape[1:]
    if nle == 1 or P == 1:
        return x.reshape(nle * P * cap, *tail)
    return x.view(P, nle, cap, *tail).transpose(0, 1).reshape(nle * P * cap, *tail)


def expert_to_rank_major(x: torch.Tensor, P: int, nle: int, cap: int) -> torch.Tensor:
    tail = x.shape[1:]
    if nle == 1 or P == 1:
        return x.reshape(P * nle * cap, *tail)
    return x.view(nle, P, cap, *tail).transpose(0, 1).reshape(P * nle * cap, *tail)


class MoEForwardState:
    """What the backward pass needs from the forward pass of the expert block.

    ``pre_em`` (the FC1 pre-activation, ``[R, F or 2F]``) is the largest saved tensor of a layer.
    With ``set_recompute`` it is not kept: the first read in the backward pass runs the FC1 GEMM
    again on the saved tokens, which happens right before the activation backward needs it, i.e.
    while the combine-gradient exchange is in flight (the reference has the same memory-saving
    fallback, fluid/moe/backward.py:616-646)."""

    def __init__(self, tokens_em: torch.Tensor, probs_em: torch.Tensor, pre_em: Optional[torch.Tensor],
                 act_em: torch.Tensor):
        self.tokens_em = tokens_em          # [R, H] dispatched tokens, expert-major
        self.probs_em = probs_em            # [R] fp32
        self.act_em = act_em                # [R, F] act * prob
        self._pre_em = pre_em
        self._recompute = None

    def set_recompute(self, fn) -> None:
        self._recompute = fn

    @property
    def pre_em(self) -> Optional[torch.Tensor]:
        if self._pre_em is None and self._recompute is not None:
            self._pre_em = self._recompute()
        return self._pre_em

    @pre_em.setter
    def pre_em(self, value) -> None:
        self._pre_em = value


# ============================================================================================
# forward: dispatch + FC1
# ============================================================================================
def dispatch_fc1_forward(plan: EPPlan, permuted_tokens: torch.Tensor, permuted_probs: torch.Tensor,
                         w1: torch.Tensor, activation: str = "gelu", mode: str = "a2a",
                         save_pre: bool = True, fused_ctx=None, hidden_states=None,
                         sorted_indices=None) -> MoEForwardState:
    """Move routed tokens to their experts and run FC1 + activation x probability.

    w1: ``[nle, H, F]`` (``[nle, H, 2F]`` for swiglu).  Modes are described in the module
    docstring.  Counterpart of ``dispatch_fc1_p2p_forward`` (fluid/moe/forward.py:535-767).
    """
    P, nle, cap = plan.ep_size, plan.num_local_experts, plan.expert_capacity
    H = plan.hidden_size
    R = plan.rows_local
    Fw = w1.shape[2]
    F = Fw // 2 if activation == "swiglu" else Fw
    probs32 = permuted_probs.float()
    if P == 1:
        act, pre = gemm.grouped_gemm_act(permuted_tokens, w1, probs32, activation=activation,
                                         uniform_rows=cap, save_pre=save_pre)
        return MoEForwardState(permuted_tokens, probs32, pre, act)
    if mode == "fused":
        return fused_ctx.dispatch_fc1(plan, hidden_states, sorted_indices, probs32, w1, activation, save_pre)
    if mode == "a2a":
        recv = comm.all_to_all(permuted_tokens, plan.group)
        recv_p = comm.all_to_all(probs32, plan.group)
        tokens_em = rank_to_expert_major(recv, P, nle, cap).contiguous()
        probs_em = rank_to_expert_major(recv_p, P, nle, cap).contiguous()
        act, pre = gemm.grouped_gemm_act(tokens_em, w1, probs_em, activation=activation,
                                         uniform_rows=P * cap, save_pre=save_pre)
        return MoEForwardState(tokens_em, probs_em, pre, act)
    assert mode == "p2p", mode
    # ---- round-ordered pairwise exchange, FC1 of block r-1 overlaps the exchange of block r ----
    dev, dt = permuted_tokens.device, permuted_tokens.dtype
    sched = get_backward_scheduler()
    backend = get_p2p_backend()
    ctx = plan.overlap_ctx
    comm_stream = ctx.comm_stream if ctx is not None else None
    tag = f"L{plan.layer_id}"
    tokens_em = backend.alloc_recv_buffer(f"moe_tokens_{tag}", R * H, dt, dev, group=plan.group).view(R, H)
    probs_em = backend.alloc_recv_buffer(f"moe_probs_{tag}", R, torch.float32, dev, group=plan.group)
    act = torch.empty(R, F, dtype=dt, device=dev)
    pre = torch.empty(R, Fw, dtype=dt, device=dev) if save_pre else None
    me = plan.ep_rank
    t4 = tokens_em.view(nle, P, cap, H)
    p3 = probs_em.view(nle, P, cap)
    send_t = permuted_tokens.view(P, nle, cap, H)
    send_p = probs32.view(P, nle, cap)
    t4[:, me].copy_(send_t[me])
    p3[:, me].copy_(send_p[me])
    cur = current_stream(dev)
    if ctx is not None:
        ctx.data_ready_event.record(cur)
        comm_stream.wait_event(ctx.data_ready_event)
    prof = get_overhead_profiler()

    def run_block(src):
        rows, offs = plan.block(src)
        gemm.grouped_gemm_act(tokens_em, w1, probs_em, activation=activation, group_rows=rows,
                              group_offs=offs, save_pre=save_pre, act_out=act, pre_out=pre)

    t0 = sched.begin_fwd_comm(comm_stream) if ctx is not None else None
    events = []
    prev = me
    for rnd, q in enumerate(plan.partners):
        tok = prof.enter("overhead.fwd_tournament_round")
        ev = ctx.get_round_event(plan.dispatch_event_name(rnd), rnd) if ctx is not None else None
        gq = plan.global_ranks[q]
        # one message per local expert lands directly in its expert-major slot (no re-layout)
        for j in range(nle):
            last = j == nle - 1
            backend.exchange(send_t[q, j], t4[j, q], gq, q, plan.group, comm_stream, None)
            backend.exchange(send_p[q, j], p3[j, q], gq, q, plan.group, comm_stream, ev if last else None)
        events.append(ev)
        prof.exit(tok)
        # compute on the block that is already here while this exchange is in flight
        if prev != me and events[rnd - 1] is not None:
            sched.record_fwd_wait("r3_f", events[rnd - 1])
        run_block(prev)
        prev = q
    if events and events[-1] is not None:
        sched.record_fwd_wait("r3_f", events[-1])
    if ctx is not None:
        sched.end_fwd_comm("r3_f", t0, comm_stream)
    run_block(prev)
    if backend.needs_final_wait():
        backend.final_wait()
    return MoEForwardState(tokens_em, probs_em, pre, act)


# ============================================================================================
# forward: FC2 + combine
# ============================================================================================
def fc2_combine_forward(plan: EPPlan, state: MoEForwardState, w2: torch.Tensor, mode: str = "a2a",
                        fused_ctx=None) -> torch.Tensor:
    """FC2 on the expert-major activations, results returned to the owners of the tokens.

    Returns ``combined [E * cap, H]`` in permuted order (the order of ``sorted_indices``).
    Counterpart of ``fc2_combine_p2p_forward`` (fluid/moe/forward.py:774-1056).
    """
    P, nle, cap = plan.ep_size, plan.num_local_experts, plan.expert_capacity
    H = plan.hidden_size
    act = state.act_em
    if P == 1:
        return gemm.grouped_gemm(act, w2, b_layout="kn", uniform_rows=cap)
    if mode == "fused":
        return fused_ctx.fc2_combine(plan, state, w2)
    if mode == "a2a":
        out_em = gemm.grouped_gemm(act, w2, b_layout="kn", uniform_rows=P * cap)
        send = expert_to_rank_major(out_em, P, nle, cap).contiguous()
        return comm.all_to_all(send, plan.group)
    assert mode == "p2p", mode
    dev, dt = act.device, act.dtype
    sched = get_backward_scheduler()
    backend = get_p2p_backend()
    ctx = plan.overlap_ctx
    comm_stream = ctx.comm_stream if ctx is not None else None
    me = plan.ep_rank
    out_em = torch.empty(plan.rows_local, H, dtype=dt, device=dev)
    o4 = out_em.view(nle, P, cap, H)
    combined = backend.alloc_recv_buffer(f"moe_combined_L{plan.layer_id}", P * plan.S * H, dt, dev,
                                         group=plan.group).view(P * plan.S, H)
    c4 = combined.view(P, nle, cap, H)
    cur = current_stream(dev)
    prof = get_overhead_profiler()

    def run_block(src):
        rows, offs = plan.block(src)
        gemm.grouped_gemm(act, w2, b_layout="kn", group_rows=rows, group_offs=offs, out=out_em)

    order = plan.partners + [me]           # peers first so their results leave early, local last
    run_block(order[0])
    t0 = sched.begin_fwd_comm(comm_stream) if ctx is not None else None
    last_ev = None
    for rnd, q in enumerate(plan.partners):
        tok = prof.enter("overhead.fwd_tournament_round")
        ready = ctx.get_round_event("moe_fc2_ready", rnd) if ctx is not None else None
        if ready is not None:
            ready.record(cur)
            comm_stream.wait_event(ready)
        ev = ctx.get_round_event(plan.combine_event_name(rnd), rnd) if ctx is not None else None
        gq = plan.global_ranks[q]
        for j in range(nle):
            backend.exchange(o4[j, q], c4[q, j], gq, q, plan.group, comm_stream,
                             ev if j == nle - 1 else None)
        last_ev = ev
        prof.exit(tok)
        run_block(order[rnd + 1])
    c4[me].copy_(o4[:, me])
    if last_ev is not None:
        sched.record_fwd_wait("r4_f", last_ev)
    if ctx is not None:
        sched.end_fwd_comm("r4_f", t0, comm_stream)
    if backend.needs_final_wait():
        backend.final_wait()
    return combined


# ============================================================================================
# backward chunk planning
# ============================================================================================
def decompose_chunks(num_chunks: int, num_local_experts: int, capacity: int) -> Tuple[int, int]:
    """Split a backward region into ``C_expert * C_cap`` chunks: expert dimension first (largest
    divisor of nle not above the request), then the capacity dimension (largest divisor of cap not
    above what is left).  Counterpart of ``_decompose_chunks`` (fluid/moe/backward.py:143-180)."""
    c = max(1, int(num_chunks))
    ce = 1
    for cand in range(min(c, num_local_experts), 0, -1):
        if num_local_experts % cand == 0:
            ce = cand
            break
    cc = max(1, c // ce)
    while cc > 1 and capacity % cc != 0:
        cc -= 1
    return ce, cc


@dataclass
class RegionChunkConfig:
    num_chunks: int
    c_expert: int
    c_cap: int
    mode: str            # 'expert' | 'hybrid' | 'cap' | 'none'
    skip_index: bool     # one whole expert per chunk: rows are already contiguous


def build_region_chunk_config(num_chunks: int, nle: int, cap: int) -> RegionChunkConfig:
    ce, cc = decompose_chunks(num_chunks, nle, cap)
    n = ce * cc
    if n == 1:
        mode = "none"
    elif cc == 1:
        mode = "expert"
    elif ce == 1:
        mode = "cap"
    else:
        mode = "hybrid"
    return RegionChunkConfig(n, ce, cc, mode, skip_index=(cc == 1 and nle // ce == 1))


def build_moe_chunk_config(moe_combine_chunks: int, moe_dispatch_chunks: int, nle: int, cap: int) -> Dict[str, RegionChunkConfig]:
    """Chunk configuration of the two MoE backward regions (fluid/moe/backward.py:183-255)."""
    return {"moe_combine": build_region_chunk_config(moe_combine_chunks, nle, cap),
            "moe_dispatch": build_region_chunk_config(moe_dispatch_chunks, nle, cap)}


def _chunk_blocks(plan: EPPlan, cfg: RegionChunkConfig, c: int):
    """Rows of chunk ``c`` in the expert-major buffer as (group_rows, group_offs, expert_of_group)
    plus the matching view selectors for the permuted (sender-side) layout."""
    P, nle, cap = plan.ep_size, plan.num_local_experts, plan.expert_capacity
    ie, ic = divmod(c, cfg.c_cap)
    e_per = nle // cfg.c_expert
    cc = cap // cfg.c_cap
    return range(ie * e_per, (ie + 1) * e_per), slice(ic * cc, (ic + 1) * cc), cc


# ============================================================================================
# backward R1: combine-grad all-to-all + FC2 dX + activation backward
# ============================================================================================
def combine_fc2_backward(plan: EPPlan, grad_combined: torch.Tensor, state: MoEForwardState,
                         w2: torch.Tensor, activation: str, num_chunks: int = 1,
                         mode: str = "a2a", fused_ctx=None):
    """Region ``moe_combine``.  ``grad_combined [E*cap, H]`` is the gradient of the combine
    buffer in permuted order.  Returns ``(dfc2_em [R,H], dpre_em [R,Fw], dprobs_em [R] fp32)``.

    With more than one chunk the all-to-alls of all chunks are submitted up front and the FC2
    input-gradient GEMM of chunk c runs as soon as chunk c has arrived, while deferred
    weight-gradient tasks of later layers fill the first wait
    (fluid/moe/backward.py:653-1068).
    """
    P, nle, cap = plan.ep_size, plan.num_local_experts, plan.expert_capacity
    H = plan.hidden_size
    sched = get_backward_scheduler()
    sched.begin_region("moe_combine")
    try:
        if P == 1:
            sched.execute_dw_tasks(max_defer_tasks=2) if sched.is_enabled() else None
            dpre, dprobs = gemm.grouped_gemm_dact(grad_combined, w2, state.pre_em, state.probs_em,
                                                  activation=activation, uniform_rows=cap)
            return grad_combined, dpre, dprobs
        if mode == "fused":
            return fused_ctx.combine_fc2_backward(plan, grad_combined, state, w2, activation)
        cfg = build_region_chunk_config(num_chunks, nle, cap)
        dev, dt = grad_combined.device, grad_combined.dtype
        R = plan.rows_local
        if cfg.num_chunks == 1 or not sched.is_enabled():
            recv = comm.all_to_all(grad_combined, plan.group)
            dfc2 = rank_to_expert_major(recv, P, nle, cap).contiguous()
            if sched.is_enabled():
                sched.execute_dw_tasks(max_defer_tasks=2)
            dpre, dprobs = gemm.grouped_gemm_dact(dfc2, w2, state.pre_em, state.probs_em,
                                                  activation=activation, uniform_rows=P * cap)
            return dfc2, dpre, dprobs
        dfc2 = torch.empty(R, H, dtype=dt, device=dev)
        d4 = dfc2.view(nle, P, cap, H)
        g4 = grad_combined.view(P, nle, cap, H)
        dpre = torch.empty_like(state.pre_em)
        dprobs = torch.zeros(R, dtype=torch.float32, device=dev)
        tasks = []
        for c in range(cfg.num_chunks):
            experts, sl, cc = _chunk_blocks(plan, cfg, c)
            send = g4[:, experts.start:experts.stop, sl].contiguous()     # [P, e_per, cc, H]
            tasks.append((sched.submit_alltoall_call(comm.all_to_all, send, plan.group), experts, sl, cc))
        sched.execute_dw_tasks(max_defer_tasks=2)
        for tid, experts, sl, cc in tasks:
            recv = sched.wait_alltoall(tid)
            e_per = experts.stop - experts.start
            d4[experts.start:experts.stop, :, sl].copy_(recv.view(P, e_per, cc, H).transpose(0, 1))
            rows = torch.full((e_per * P,), cc, dtype=torch.int32, device=dev)
            offs = torch.tensor([(j * P + r) * cap + sl.start for j in experts for r in range(P)],
                                dtype=torch.int32, device=dev)
            _dact_blocks(dfc2, w2, state, activation, rows, offs, experts, P, dpre, dprobs)
        return dfc2, dpre, dprobs
    finally:
        sched.end_region()


def _dact_blocks(dfc2, w2, state, activation, rows, offs, experts, P, dpre, dprobs):
    """FC2 dX + activation backward on a set of row blocks; block b belongs to expert
    ``experts[b // P]`` (passed to the kernel as the group -> weight map)."""
    group_b = torch.tensor([j for j in experts for _ in range(P)], dtype=torch.int32, device=w2.device)
    gemm.grouped_gemm_dact(dfc2, w2, state.pre_em, state.probs_em, activation=activation,
                           group_rows=rows, group_offs=offs, group_b=group_b, dpre_out=dpre,
                           dprobs_out=dprobs)


# ============================================================================================
# backward R2: FC1 dX + dispatch-grad all-to-all
# ============================================================================================
def fc1_dispatch_backward(plan: EPPlan, dpre_em: torch.Tensor, w1: torch.Tensor,
                          num_chunks: int = 1, mode: str = "a2a", fused_ctx=None,
                          dprobs_em: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Region ``moe_dispatch``: ``dTok = dpre @ W1^T`` per expert, sent back to the token owners.
    Returns the gradient of the permuted tokens ``[E*cap, H]`` (fluid/moe/backward.py:1075-1411).
    """
    P, nle, cap = plan.ep_size, plan.num_local_experts, plan.expert_capacity
    H = plan.hidden_size
    sched = get_backward_scheduler()
    sched.begin_region("moe_dispatch")
    try:
        if P == 1:
            out = gemm.grouped_gemm(dpre_em, w1, b_layout="nk", uniform_rows=cap)
            if sched.is_enabled():
                sched.execute_dw_tasks(max_defer_tasks=2)
            return out
        if mode == "fused":
            return fused_ctx.fc1_dispatch_backward(plan, dpre_em, w1, dprobs_em)
        cfg = build_region_chunk_config(num_chunks, nle, cap)
        dev, dt = dpre_em.device, dpre_em.dtype
        if cfg.num_chunks == 1 or not sched.is_enabled():
            dtok = gemm.grouped_gemm(dpre_em, w1, b_layout="nk", uniform_rows=P * cap)
            send = expert_to_rank_major(dtok, P, nle, cap).contiguous()
            if sched.is_enabled():
                tid = sched.submit_alltoall_call(comm.all_to_all, send, plan.group)
                sched.execute_dw_tasks(max_defer_tasks=2)
                return sched.wait_alltoall(tid)
            return comm.all_to_all(send, plan.group)
        dtok = torch.empty(plan.rows_local, H, dtype=dt, device=dev)
        t4 = dtok.view(nle, P, cap, H)
        out = torch.empty(P * plan.S, H, dtype=dt, device=dev)
        o4 = out.view(P, nle, cap, H)
        tasks = []
        for c in range(cfg.num_chunks):
            experts, sl, cc = _chunk_blocks(plan, cfg, c)
            e_per = experts.stop - experts.start
            rows = torch.full((e_per * P,), cc, dtype=torch.int32, device=dev)
            offs = torch.tensor([(j * P + r) * cap + sl.start for j in experts for r in range(P)],
                                dtype=torch.int32, device=dev)
            group_b = torch.tensor([j for j in experts for _ in range(P)], dtype=torch.int32, device=dev)
            gemm.grouped_gemm(dpre_em, w1, b_layout="nk", group_rows=rows, group_offs=offs,
                              group_b=group_b, out=dtok)
            send = t4[experts.start:experts.stop, :, sl].transpose(0, 1).contiguous()  # [P,e_per,cc,H]
            tasks.append((sched.submit_alltoall_call(comm.all_to_all, send, plan.group), experts, sl, cc))
        sched.execute_dw_tasks(max_defer_tasks=2)
        for tid, experts, sl, cc in tasks:
            recv = sched.wait_alltoall(tid)
            e_per = experts.stop - experts.start
            o4[:, experts.start:experts.stop, sl].copy_(recv.view(P, e_per, cc, H))
        return out
    finally:
        sched.end_region()


# ============================================================================================
# weight-gradient tasks
# ============================================================================================
def recompute_fc1_gemm(all_expert_tokens: torch.Tensor, all_tokens_per_expert, weight1: torch.Tensor) -> torch.Tensor:
    """FC1 pre-activations again from the dispatched tokens: ``tokens_e @ weight1[e]`` for every
    local expert e, rows of expert e being the next ``all_tokens_per_expert[e]`` rows
    (fluid/moe/backward.py:616-646).  The layer itself recomputes through
    ``MoEForwardState.pre_em``; this is the stand-alone form of the same GEMM."""
    counts = [int(n) for n in all_tokens_per_expert]
    if all_expert_tokens.shape[0] == 0:
        return all_expert_tokens.new_empty(0, weight1.shape[-1])
    dev = all_expert_tokens.device
    rows = torch.tensor(counts, dtype=torch.int32, device=dev)
    offs = torch.tensor([sum(counts[:i]) for i in range(len(counts))], dtype=torch.int32, device=dev)
    return gemm.grouped_gemm(all_expert_tokens, weight1.detach(), b_layout="kn", group_rows=rows, group_offs=offs)


def skip_all_dw() -> bool:
    """Ablation ``FLUID_SKIP_ALL_DW=1``: deferrable weight-gradient tasks run only at the end of the
    backward pass, in no communication window (fluid/moe/backward.py:361-363)."""
    return bool(get_backward_scheduler().skip_all_dw)


def skip_dispatch_dw() -> bool:
    """Ablation ``FLUID_SKIP_DISPATCH_DW=1``: none of them in the window of the dispatch-gradient
    exchange (fluid/moe/backward.py:366-368)."""
    return bool(get_backward_scheduler().skip_dispatch_dw)


def fused_optimizer_of(param, sched):
    """The optimizer that wants to run in this parameter's weight-gradient epilogue, or None.
    Only taken on the first (and only) gradient write of a step, when the parameter has no
    expert-data-parallel replicas."""
    fa = getattr(param, "_fused_adam", None)
    if fa is None or getattr(param, "_ar_buf_written", False):
        return None
    if getattr(sched, "expert_dp_world", 1) > 1:
        return None
    return fa


def register_moe_dw_tasks(plan: EPPlan, state: MoEForwardState, dfc2_em: torch.Tensor,
                          dpre_em: torch.Tensor, w1_param, w2_param, layer_id: int = 0,
                          layer_name: str = "moe", which: str = "both") -> None:
    """Queue ``dW2[e] = actW[e]^T dFC2out[e]`` and ``dW1[e] = tokens[e]^T dFC1[e]``
    (fluid/moe/backward.py:487-613).  When the parameter lives in a flat gradient buffer the GEMM
    accumulates straight into its fp32 slice; when an optimizer asked to run in the epilogue
    (``FusedAdam.fuse_into_backward``) the GEMM updates the parameter instead and stores nothing.
    ``which`` selects the tasks to queue: a parameter that is updated in place may only be queued
    once its last use of this backward pass (the FC1 dX GEMM for ``w1``) has been issued."""
    sched = get_backward_scheduler()
    nle = plan.num_local_experts
    rows_per = plan.ep_size * plan.expert_capacity if plan.ep_size > 1 else plan.expert_capacity
    max_ctas = sched.dw_max_ctas

    def make(a, dy, param):
        def run():
            fa = fused_optimizer_of(param, sched) if sched.is_enabled() else None
            gscale = 1.0 / max(1, sched.shared_dp_world)
            if fa is not None and getattr(fa, "fused_mode", "epilogue") == "epilogue":
                fa.wgrad_update(param, a, dy, nle, grad_scale=gscale, uniform_rows=rows_per, max_ctas=max_ctas)
                return None
            buf = sched._buffer_of(param) if sched.is_enabled() else None
            if buf is not None and param.main_grad.dtype == torch.float32 and a.is_cuda:
                first = not getattr(param, "_ar_buf_written", False)
                gemm.grouped_gemm_wgrad(a, dy, nle, uniform_rows=rows_per, out=param.main_grad,
                                        accumulate=not first, alpha=gscale if fa is not None else 1.0,
                                        max_ctas=max_ctas)
                if fa is not None:
                    fa.update_on_stream(param)     # Adam for this parameter behind the GEMM, on a side stream
                return None
            return gemm.grouped_gemm_wgrad(a, dy, nle, uniform_rows=rows_per, alpha=gscale if fa is not None else 1.0)
        return run

    if which in ("both", "w2"):
        sched.register_dw_task(f"{layer_name}.w2", layer_id, make(state.act_em, dfc2_em, w2_param), w2_param)
    if which in ("both", "w1"):
        sched.register_dw_task(f"{layer_name}.w1", layer_id, make(state.tokens_em, dpre_em, w1_param), w1_param)


# ============================================================================================
# baseline module (the oracle of the correctness tests)
# ============================================================================================
class MoEBaseline(nn.Module):
    """Plain expert-parallel MoE: router -> permute -> all-to-all -> experts -> all-to-all ->
    un-permute, differentiated by autograd.  It is the comparison baseline of the overlap paths
    and runs on CPU/gloo as well as on GPUs.  (Named in the reference's README:47; its code is
    not part of the reference tree.)"""

    def __init__(self, hidden_size: int, ffn_hidden_size: int, num_experts: int, top_k: int,
                 ep_group=None, activation: str = "gelu", capacity_factor: float = 1.0,
                 router_dtype=torch.float32, dtype=torch.float32, device=None, init_std: float = 0.02):
        super().__init__()
        self.hidden_size, self.ffn, self.num_experts, self.top_k = hidden_size, ffn_hidden_size, num_experts, top_k
        self.ep_group = ep_group
        self.P = comm.group_size(ep_group)
        self.nle = num_experts // self.P
        self.activation, self.capacity_factor, self.router_dtype = activation, capacity_factor, router_dtype
        fw = 2 * ffn_hidden_size if activation == "swiglu" else ffn_hidden_size
        self.router_weight = nn.Parameter(torch.randn(hidden_size, num_experts, dtype=dtype, device=device) * init_std)
        self.moe_w1 = nn.Parameter(torch.randn(self.nle, hidden_size, fw, dtype=dtype, device=device) * init_std)
        self.moe_w2 = nn.Parameter(torch.randn(self.nle, ffn_hidden_size, hidden_size, dtype=dtype, device=device) * init_std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: [T, H] -> [T, H]."""
        T, H = x.shape
        P, nle, E, k = self.P, self.nle, self.num_experts, self.top_k
        logits = x.to(self.router_dtype) @ self.router_weight.to(self.router_dtype)
        top_logits, top_idx = torch.topk(logits, k, dim=-1)
        top_probs = torch.softmax(top_logits, dim=-1, dtype=torch.float32)
        cap = router_ops.expert_capacity(T, k, E, self.capacity_factor)
        with torch.no_grad():
            plan = router_ops.build_padded_plan(top_idx, top_probs.detach(), E, cap)
        # differentiable slot probabilities: gather from the (T, k) probabilities
        slots = plan.slot_of_token.long()
        flat_probs = torch.zeros(E * cap + 1, dtype=torch.float32, device=x.device)
        flat_probs = flat_probs.scatter(0, torch.where(slots >= 0, slots, torch.full_like(slots, E * cap)).reshape(-1),
                                        top_probs.reshape(-1))[: E * cap]
        permuted = x.index_select(0, plan.sorted_indices)
        recv = _A2A.apply(permuted, self.ep_group)
        recv_p = _A2A.apply(flat_probs, self.ep_group)
        tok = rank_to_expert_major(recv, P, nle, cap).view(nle, P * cap, H)
        prb = rank_to_expert_major(recv_p, P, nle, cap).view(nle, P * cap, 1)
        outs = []
        for j in range(nle):
            h = tok[j].float() @ self.moe_w1[j].float()
            a = gemm.act_ref(h, self.activation) * prb[j]
            outs.append((a @ self.moe_w2[j].float()).to(x.dtype))
        out_em = torch.stack(outs, 0).view(nle * P * cap, H)
        back = _A2A.apply(expert_to_rank_major(out_em, P, nle, cap).contiguous(), self.ep_group)
        out = torch.zeros(T, H, dtype=back.dtype, device=x.device)
        return out.index_add(0, plan.sorted_indices, back)


class _A2A(torch.autograd.Function):
    """Equal-split all-to-all with its own transpose as the backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return comm.all_to_all(x.contiguous(), group)

    @staticmethod
    def backward(ctx, g):
        return comm.all_to_all(g.contiguous(), ctx.group), None


# ============================================================================================
# README-era functional entry point
# ============================================================================================
def moe_multicard_p2p_overlap_forward(tokens: torch.Tensor, input_splits, output_splits,
                                      weight1: torch.Tensor, weight2: torch.Tensor, ep_group,
                                      activation_func="gelu", overlap_ctx: Optional[MultiCardOverlapContext] = None,
                                      layer_id: int = 0, num_local_experts: Optional[int] = None,
                                      tokens_per_expert: Optional[torch.Tensor] = None,
                                      num_global_tokens_per_local_expert: Optional[torch.Tensor] = None,
                                      probs: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Expert computation for already-permuted ``tokens`` with pairwise-overlapped exchange.

    ``tokens [sum(input_splits), H]`` is ordered by destination rank, and within a rank by local
    expert; ``input_splits[p]`` rows go to EP rank p and ``output_splits[p]`` rows come from it.
    ``num_global_tokens_per_local_expert [P, nle]`` gives, for every source rank, how many of its
    rows belong to each of this rank's experts (required unless every split is uniform, in which
    case rows are divided evenly between the local experts).  Returns the expert outputs in the
    order of ``tokens``.  Signature from the reference's README:62-67; both uniform (padded) and
    variable (dropless) splits are accepted.
    """
    P = comm.group_size(ep_group)
    me = comm.group_rank(ep_group)
    nle = num_local_experts if num_local_experts is not None else weight1.shape[0]
    act = activation_func if isinstance(activation_func, str) else getattr(activation_func, "__name__", "gelu")
    act = {"gelu": "gelu", "silu": "silu", "swiglu": "swiglu"}.get(act, "gelu")
    H = tokens.shape[1]
    dev = tokens.device
    input_splits = [int(s) for s in input_splits]
    output_splits = [int(s) for s in output_splits]
    if num_global_tokens_per_local_expert is None:
        assert all(s % nle == 0 for s in output_splits), "per-expert counts are needed for uneven splits"
        counts = torch.tensor([[s // nle] * nle for s in output_splits], dtype=torch.int64)
    else:
        counts = num_global_tokens_per_local_expert.to("cpu", torch.int64).view(P, nle)
    backend = get_p2p_backend()
    comm_stream = overlap_ctx.comm_stream if overlap_ctx is not None else None
    partners = overlap_ctx.partners_in_order(me) if (overlap_ctx is not None and P > 1) else \
        [(me + i) % P for i in range(1, P)]
    ranks = dist.get_process_group_ranks(ep_group) if (ep_group is not None and dist.is_initialized()) else list(range(P))
    in_offs = [0]
    for s in input_splits:
        in_offs.append(in_offs[-1] + s)
    results = [None] * P

    def experts_on(block: torch.Tensor, src: int, p_block: Optional[torch.Tensor]):
        rows = counts[src].to(torch.int32)
        offs = torch.cumsum(rows, 0, dtype=torch.int32) - rows
        rows_d, offs_d = rows.to(dev), offs.to(dev)
        a, _ = gemm.grouped_gemm_act(block, weight1, p_block, activation=act, group_rows=rows_d,
                                     group_offs=offs_d, save_pre=False)
        return gemm.grouped_gemm(a, weight2, b_layout="kn", group_rows=rows_d, group_offs=offs_d)

    cur = current_stream(dev)
    if overlap_ctx is not None:
        overlap_ctx.data_ready_event.record(cur)
        comm_stream.wait_event(overlap_ctx.data_ready_event)
    recv_bufs, recv_probs, evs = {}, {}, {}
    for rnd, q in enumerate(partners):
        ev = overlap_ctx.get_round_event(f"moe_fn_dispatch_{layer_id}", rnd) if overlap_ctx is not None else None
        rb = torch.empty(output_splits[q], H, dtype=tokens.dtype, device=dev)
        backend.exchange(tokens[in_offs[q]:in_offs[q + 1]], rb, ranks[q], q, ep_group, comm_stream,
                         None if probs is not None else ev)
        if probs is not None:
            pb = torch.empty(output_splits[q], dtype=torch.float32, device=dev)
            backend.exchange(probs[in_offs[q]:in_offs[q + 1]].float().contiguous(), pb, ranks[q], q,
                             ep_group, comm_stream, ev)
            recv_probs[q] = pb
        recv_bufs[q], evs[q] = rb, ev
    local = tokens[in_offs[me]:in_offs[me + 1]]
    local_p = probs[in_offs[me]:in_offs[me + 1]].float().contiguous() if probs is not None else None
    results[me] = experts_on(local, me, local_p)
    out = torch.empty_like(tokens)
    out[in_offs[me]:in_offs[me + 1]] = results[me]
    back_evs = []
    for rnd, q in enumerate(partners):
        if evs[q] is not None:
            cur.wait_event(evs[q])
        res = experts_on(recv_bufs[q], q, recv_probs.get(q))
        ready = overlap_ctx.get_round_event(f"moe_fn_ready_{layer_id}", rnd) if overlap_ctx is not None else None
        if ready is not None:
            ready.record(cur)
            comm_stream.wait_event(ready)
        ev = overlap_ctx.get_round_event(f"moe_fn_combine_{layer_id}", rnd) if overlap_ctx is not None else None
        backend.exchange(res, out[in_offs[q]:in_offs[q + 1]], ranks[q], q, ep_group, comm_stream, ev)
        back_evs.append(ev)
    for ev in back_evs:
        if ev is not None:
            cur.wait_event(ev)
    if backend.needs_final_wait():
        backend.final_wait()
    return out


def pad_moe_dispatch(tokens: torch.Tensor, tokens_per_expert: torch.Tensor, capacity: int,
                     probs: Optional[torch.Tensor] = None):
    """Pad or truncate every expert's run of rows to exactly ``capacity`` rows.

    ``tokens [sum(tokens_per_expert), H]`` is expert-major with variable counts; the result is
    ``[E * capacity, H]`` with zero rows (and zero probabilities) as padding.  Vectorised, no host
    synchronisation (fluid/moe/forward.py:1059-1125)."""
    E = tokens_per_expert.numel()
    dev = tokens.device
    counts = tokens_per_expert.to(dev, torch.int64)
    starts = torch.cumsum(counts, 0) - counts
    slot = torch.arange(capacity, device=dev).unsqueeze(0).expand(E, capacity)
    valid = slot < counts.unsqueeze(1)
    src = (starts.unsqueeze(1) + slot).clamp(max=max(tokens.shape[0] - 1, 0))
    out = tokens.index_select(0, src.reshape(-1)) * valid.reshape(-1, 1).to(tokens.dtype)
    if probs is None:
        return out, valid.reshape(-1)
    return out, probs.index_select(0, src.reshape(-1)) * valid.reshape(-1).to(probs.dtype), valid.reshape(-1)


# ============================================================================================
# router backward (functional form of the code used inside the layer)
# ============================================================================================
def router_backward(grad_permuted_probs: torch.Tensor, plan_or_sorted_indices, top_indices: torch.Tensor,
                    top_probs: torch.Tensor, router_logits: torch.Tensor, router_weight: torch.Tensor,
                    num_experts: int, aux_loss_coeff: float = 0.0, z_loss_coeff: float = 0.0,
                    cp_group=None, out_dtype: Optional[torch.dtype] = None):
    """Gradient of the router: returns ``(d_hidden [T, H], d_logits [T, E] fp32)``.

    ``grad_permuted_probs`` is the gradient of every slot's probability in permuted order;
    ``plan_or_sorted_indices`` is the :class:`RoutingPlan` of the forward pass.  The load-balancing
    loss uses the per-expert token counts summed over the sequence-parallel group
    (fluid/moe/backward.py:1419-1532)."""
    rplan = plan_or_sorted_indices
    T = top_indices.shape[0]
    tpe = None
    world = comm.group_size(cp_group) if cp_group is not None else 1
    if aux_loss_coeff > 0.0:
        tpe = rplan.routed_per_expert.float()
        if world > 1:
            dist.all_reduce(tpe, group=cp_group)
    dlogits = router_ops.router_backward_logits(grad_permuted_probs, rplan, top_indices, top_probs,
                                                router_logits, num_experts, aux_loss_coeff, z_loss_coeff,
                                                tpe, T * world)
    w = router_weight.detach()
    dx = dlogits.to(w.dtype) @ w.t()
    return (dx.to(out_dtype) if out_dtype is not None else dx), dlogits


def register_router_dw_task(layer_id: int, hidden_states: torch.Tensor, d_logits: torch.Tensor,
                            router_weight_param, layer_name: str = "router") -> None:
    """Queue ``dWr = hidden^T @ dLogits`` (fluid/moe/backward.py:1535-1578)."""
    sched = get_backward_scheduler()
    sched.register_dw_task(layer_name, layer_id,
                           lambda: hidden_states.float().t() @ d_logits.float(), router_weight_param)


# names used by the reference for the same entry points
dispatch_fc1_p2p_forward = dispatch_fc1_forward
fc2_combine_p2p_forward = fc2_combine_forward
