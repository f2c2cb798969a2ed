"""Ulysses sequence-parallel attention: QKV projection + SP->HP exchange, HP->SP exchange +
output projection, and the two backward regions.

Each rank holds a contiguous block of ``s_local = s / P`` positions.  The QKV weight rows are
grouped by KV group ``[g][q_0 .. q_{qpg-1} | k | v]`` (``d`` rows each), rank p attends with the
heads of groups ``[p*G, (p+1)*G)`` over the *full* sequence, and the output-projection columns are
ordered by global head, i.e. by owning rank (fluid/attention/forward.py:172-189,393).

Transports: ``a2a`` (one all-to-all per exchange), ``p2p`` (round-ordered pairwise exchanges
overlapped with the per-peer GEMM slices, fluid/attention/forward.py:220-261,435-476) and ``fused``
(GEMM epilogues store straight into the peers' buffers).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import gemm
from ..parallel import comm
from ..parallel.p2p_backend import get_p2p_backend
from ..parallel.scheduler import get_backward_scheduler
from ..parallel.schedule import MultiCardOverlapContext
from ..parallel.streams import current_stream
from ..utils.overhead_profiler import get_overhead_profiler


class CPPlan:
    """Static description of the Ulysses exchange of one layer (fluid/attention/forward.py:42-127)."""

    def __init__(self, seq_local: int, batch: int, hidden_size: int, num_heads: int,
                 num_kv_heads: int, head_dim: int, cp_group=None, dtype=torch.bfloat16, device=None,
                 overlap_ctx: Optional[MultiCardOverlapContext] = None):
        self.group = cp_group
        self.cp_size = P = comm.group_size(cp_group)
        self.cp_rank = comm.group_rank(cp_group)
        assert num_heads % num_kv_heads == 0 and num_kv_heads % P == 0 and num_heads % P == 0, \
            (num_heads, num_kv_heads, P)
        self.seq_local, self.batch, self.hidden_size = seq_local, batch, hidden_size
        self.seq_full = seq_local * P
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.q_per_group = num_heads // num_kv_heads
        self.group_size = (self.q_per_group + 2) * head_dim          # QKV columns of one KV group
        self.groups_per_rank = num_kv_heads // P
        self.proj_per_rank = self.groups_per_rank * self.group_size   # QKV columns owned by a rank
        self.heads_per_rank = num_heads // P
        self.attn_per_rank = self.heads_per_rank * head_dim           # attention-output columns
        self.dtype, self.device = dtype, device
        self.overlap_ctx = overlap_ctx
        self.layer_id = 0
        if overlap_ctx is not None and P > 1:
            self.partners = overlap_ctx.partners_in_order(self.cp_rank)
        else:
            self.partners = [(self.cp_rank + i) % P for i in range(1, P)]
        self.global_ranks = (dist.get_process_group_ranks(cp_group)
                             if (cp_group is not None and dist.is_initialized()) else list(range(P)))
        self.weight_row_offsets = [p * self.proj_per_rank for p in range(P)]
        self.recv_seq_starts = [p * seq_local for p in range(P)]

    def signature(self):
        return (self.seq_local, self.batch, self.hidden_size, self.num_heads, self.num_kv_heads,
                self.head_dim, self.cp_size)


def split_qkv(qkv_full: torch.Tensor, plan: CPPlan):
    """``[s, b, G, gs] -> q [s,b,G*qpg,d] (a copy when G > 1), k [s,b,G,d], v [s,b,G,d]`` (views)."""
    s, b = qkv_full.shape[0], qkv_full.shape[1]
    G, qpg, d = plan.groups_per_rank, plan.q_per_group, plan.head_dim
    h = qkv_full.view(s, b, G, qpg + 2, d)
    return h[:, :, :, :qpg].reshape(s, b, G * qpg, d), h[:, :, :, qpg], h[:, :, :, qpg + 1]


# ============================================================================================
# forward
# ============================================================================================
def qkv_projection_forward(x: torch.Tensor, qkv_weight: torch.Tensor, plan: CPPlan,
                           mode: str = "a2a", fused_ctx=None, defer_wait: bool = False) -> torch.Tensor:
    """x ``[s_local*b, H]`` -> ``qkv_full [s, b, G, gs]`` (this rank's heads, full sequence).

    Counterpart of ``qkv_projection_p2p_forward`` (fluid/attention/forward.py:130-277).
    """
    P = plan.cp_size
    sl, b, G, gs, ppr = plan.seq_local, plan.batch, plan.groups_per_rank, plan.group_size, plan.proj_per_rank
    T = sl * b
    if P == 1:
        return gemm.gemm_nt(x, qkv_weight).view(sl, b, G, gs)
    if mode == "fused":
        return fused_ctx.qkv_sp2hp(x, qkv_weight, plan, defer_wait)
    if mode == "a2a":
        full = gemm.gemm_nt(x, qkv_weight)                        # [T, P*ppr]
        send = full.view(sl, b, P, ppr).permute(2, 0, 1, 3).contiguous()
        out = comm.all_to_all(send.view(P * sl, b, ppr), plan.group)
        return out.view(P * sl, b, G, gs)
    assert mode == "p2p", mode
    dev, dt = x.device, x.dtype
    me = plan.cp_rank
    ctx = plan.overlap_ctx
    comm_stream = ctx.comm_stream if ctx is not None else None
    sched = get_backward_scheduler()
    backend = get_p2p_backend()
    cur = current_stream(dev)
    prof = get_overhead_profiler()
    qkv_full = backend.alloc_recv_buffer(f"attn_qkv_L{plan.layer_id}", P * sl * b * ppr, dt, dev,
                                         group=plan.group).view(P * sl, b, ppr)
    t0 = sched.begin_fwd_comm(comm_stream) if ctx is not None else None
    last_ev = None
    for rnd, q in enumerate(plan.partners):
        w_q = qkv_weight[q * ppr:(q + 1) * ppr]
        send = gemm.gemm_nt(x, w_q).view(sl, b, ppr)
        tok = prof.enter("overhead.fwd_tournament_round")
        if ctx is not None:
            ready = ctx.get_round_event("attn_qkv_ready", rnd)
            ready.record(cur)
            comm_stream.wait_event(ready)
        ev = ctx.get_round_event("attn_qkv", rnd) if ctx is not None else None
        backend.exchange(send, qkv_full[q * sl:(q + 1) * sl], plan.global_ranks[q], q, plan.group,
                         comm_stream, ev)
        last_ev = ev
        prof.exit(tok)
    gemm.gemm_nt(x, qkv_weight[me * ppr:(me + 1) * ppr], out=qkv_full[me * sl:(me + 1) * sl].view(T, ppr))
    if last_ev is not None:
        sched.record_fwd_wait("r1_f", last_ev)
    if ctx is not None:
        sched.end_fwd_comm("r1_f", t0, comm_stream)
    if backend.needs_final_wait():
        backend.final_wait()
    return qkv_full.view(P * sl, b, G, gs)


def output_projection_forward(attn_out: torch.Tensor, proj_weight: torch.Tensor, plan: CPPlan,
                              mode: str = "a2a", fused_ctx=None, residual: Optional[torch.Tensor] = None,
                              pushed: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """attn_out ``[s, b, h_local, d]`` -> ``(out [s_local*b, H], attn_input_full [s_local*b, n_h*d])``.

    ``residual`` (same shape as out) is added in the GEMM epilogue when given.
    Counterpart of ``output_projection_p2p_forward`` (fluid/attention/forward.py:332-484).
    """
    P = plan.cp_size
    sl, b, dpr = plan.seq_local, plan.batch, plan.attn_per_rank
    T = sl * b
    H = proj_weight.shape[0]

    def project(a_in, w, out=None, accumulate=False):
        return gemm.gemm_nt(a_in, w, out=out, accumulate=accumulate)

    def with_residual(a_in, w):
        if residual is None:
            return project(a_in, w)
        out = residual.clone()
        return project(a_in, w, out=out, accumulate=True)

    if P == 1:
        a_full = attn_out.reshape(T, dpr)
        return with_residual(a_full, proj_weight), a_full
    if mode == "fused":
        return fused_ctx.hp2sp_outproj(attn_out, proj_weight, plan, residual, pushed)
    if mode == "a2a":
        a_full = comm.hp2sp(attn_out, plan.group).view(T, P * dpr)
        return with_residual(a_full, proj_weight), a_full
    assert mode == "p2p", mode
    dev, dt = attn_out.device, attn_out.dtype
    me = plan.cp_rank
    ctx = plan.overlap_ctx
    comm_stream = ctx.comm_stream if ctx is not None else None
    sched = get_backward_scheduler()
    backend = get_p2p_backend()
    cur = current_stream(dev)
    prof = get_overhead_profiler()
    a_full = torch.empty(sl, b, P, dpr, dtype=dt, device=dev)
    a2 = a_full.view(T, P * dpr)
    out = residual.clone() if residual is not None else torch.zeros(T, H, dtype=dt, device=dev)
    src = attn_out.view(P, sl, b, dpr)
    if ctx is not None:
        ctx.data_ready_event.record(cur)
        comm_stream.wait_event(ctx.data_ready_event)
    t0 = sched.begin_fwd_comm(comm_stream) if ctx is not None else None
    events, staged = [], []
    for rnd, q in enumerate(plan.partners):
        tok = prof.enter("overhead.fwd_tournament_round")
        ev = ctx.get_round_event("attn_output", rnd) if ctx is not None else None
        recv = backend.alloc_recv_buffer(f"attn_out_L{plan.layer_id}_r{rnd}", sl * b * dpr, dt, dev,
                                         group=plan.group).view(sl, b, dpr)
        backend.exchange(src[q].contiguous(), recv, plan.global_ranks[q], q, plan.group, comm_stream, ev)
        events.append(ev)
        staged.append((q, recv))
        prof.exit(tok)
        if rnd == 0:
            a_full[:, :, me].copy_(src[me])
            project(a2[:, me * dpr:(me + 1) * dpr], proj_weight[:, me * dpr:(me + 1) * dpr], out=out, accumulate=True)
        else:
            pq, prev = staged[rnd - 1]
            if events[rnd - 1] is not None:
                sched.record_fwd_wait("r2_f", events[rnd - 1])
            a_full[:, :, pq].copy_(prev)
            project(a2[:, pq * dpr:(pq + 1) * dpr], proj_weight[:, pq * dpr:(pq + 1) * dpr], out=out, accumulate=True)
    pq, prev = staged[-1]
    if events[-1] is not None:
        sched.record_fwd_wait("r2_f", events[-1])
    if ctx is not None:
        sched.end_fwd_comm("r2_f", t0, comm_stream)
    a_full[:, :, pq].copy_(prev)
    project(a2[:, pq * dpr:(pq + 1) * dpr], proj_weight[:, pq * dpr:(pq + 1) * dpr], out=out, accumulate=True)
    if backend.needs_final_wait():
        backend.final_wait()
    return out, a2


# ============================================================================================
# backward
# ============================================================================================
def _valid_chunks(n: int, requested: int, what: str) -> int:
    c = max(1, int(requested))
    if n % c != 0:
        from .moe import _warn_once
        _warn_once(f"chunks:{what}:{n}:{c}", f"{what}: {n} rows do not divide into {c} chunks; using 1")
        return 1
    return c


def outproj_sp2hp_backward(d_out: torch.Tensor, proj_weight: torch.Tensor, plan: CPPlan,
                           num_chunks: int = 1, mode: str = "a2a", fused_ctx=None,
                           defer_wait: bool = False) -> torch.Tensor:
    """Region ``attn_proj``: ``dAttn = dOut @ Wproj`` per sequence chunk, each chunk sent through
    its SP->HP all-to-all while the next chunk is computed.  Returns ``[s, b, h_local, d]``.
    (fluid/attention/backward.py:46-184)"""
    P = plan.cp_size
    sl, b, dpr, d = plan.seq_local, plan.batch, plan.attn_per_rank, plan.head_dim
    hl = plan.heads_per_rank
    sched = get_backward_scheduler()
    sched.begin_region("attn_proj")
    try:
        if P == 1:
            out = gemm.gemm_nn(d_out, proj_weight).view(sl, b, hl, d)
            if sched.is_enabled():
                sched.execute_dw_tasks(max_defer_tasks=2)
            return out
        if mode == "fused":
            return fused_ctx.outproj_dx_sp2hp(d_out, proj_weight, plan, defer_wait)
        C = _valid_chunks(sl, num_chunks, "attn_proj") if sched.is_enabled() else 1
        dev, dt = d_out.device, d_out.dtype
        if C == 1:
            da = gemm.gemm_nn(d_out, proj_weight).view(sl, b, P * hl, d)
            if sched.is_enabled():
                tid = sched.submit_alltoall_call(comm.sp2hp, da, plan.group)
                sched.execute_dw_tasks(max_defer_tasks=2)
                return sched.wait_alltoall(tid)
            return comm.sp2hp(da, plan.group)
        sc = sl // C
        out = torch.empty(P, sl, b, hl, d, dtype=dt, device=dev)
        d3 = d_out.view(sl, b, -1)
        tasks = []
        for c in range(C):
            rows = d3[c * sc:(c + 1) * sc].reshape(sc * b, -1)
            da = gemm.gemm_nn(rows, proj_weight).view(sc, b, P * hl, d)
            tasks.append(sched.submit_alltoall_call(comm.sp2hp, da, plan.group))
        sched.execute_dw_tasks(max_defer_tasks=2)
        for c, tid in enumerate(tasks):
            recv = sched.wait_alltoall(tid)                      # [P*sc, b, hl, d]
            out[:, c * sc:(c + 1) * sc].copy_(recv.view(P, sc, b, hl, d))
        return out.view(P * sl, b, hl, d)
    finally:
        sched.end_region()


def hp2sp_qkv_backward(dqkv_hp: torch.Tensor, qkv_weight: torch.Tensor, plan: CPPlan,
                       num_chunks: int = 1, mode: str = "a2a", fused_ctx=None
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Region ``attn_qkv``: ``dqkv_hp [s, b, G, gs]`` goes back through the HP->SP all-to-all in
    sequence chunks; chunk c's ``dX = dQKV @ Wqkv`` runs while later chunks are in flight.
    Returns ``(dx [s_local*b, H], dqkv_sp [s_local*b, P*ppr])`` (the latter feeds the QKV weight
    gradient).  (fluid/attention/backward.py:192-376)"""
    P = plan.cp_size
    sl, b, ppr = plan.seq_local, plan.batch, plan.proj_per_rank
    T = sl * b
    sched = get_backward_scheduler()
    sched.begin_region("attn_qkv")
    try:
        if P == 1:
            dq = dqkv_hp.reshape(T, ppr)
            if sched.is_enabled():
                sched.execute_dw_tasks(max_defer_tasks=2)
            return gemm.gemm_nn(dq, qkv_weight), dq
        if mode == "fused":
            return fused_ctx.hp2sp_qkv_dx(dqkv_hp, qkv_weight, plan)
        x3 = dqkv_hp.reshape(P * sl, b, 1, ppr)                  # one "head" of width ppr per rank
        C = _valid_chunks(sl, num_chunks, "attn_qkv") if sched.is_enabled() else 1
        dev, dt = dqkv_hp.device, dqkv_hp.dtype
        if C == 1:
            if sched.is_enabled():
                tid = sched.submit_alltoall_call(comm.hp2sp, x3, plan.group)
                sched.execute_dw_tasks(max_defer_tasks=2)
                dq = sched.wait_alltoall(tid).view(T, P * ppr)
            else:
                dq = comm.hp2sp(x3, plan.group).view(T, P * ppr)
            return gemm.gemm_nn(dq, qkv_weight), dq
        sc = sl // C
        x5 = x3.view(P, sl, b, 1, ppr)
        dq_full = torch.empty(sl, b, P * ppr, dtype=dt, device=dev)
        dx = torch.empty(sl, b, qkv_weight.shape[1], dtype=dt, device=dev)
        tasks = []
        for c in range(C):
            send = x5[:, c * sc:(c + 1) * sc].reshape(P * sc, b, 1, ppr).contiguous()
            tasks.append(sched.submit_alltoall_call(comm.hp2sp, send, plan.group))
        sched.execute_dw_tasks(max_defer_tasks=2)
        for c, tid in enumerate(tasks):
            recv = sched.wait_alltoall(tid)                      # [sc, b, P, ppr]
            dq_full[c * sc:(c + 1) * sc].copy_(recv.view(sc, b, P * ppr))
            gemm.gemm_nn(dq_full[c * sc:(c + 1) * sc].view(sc * b, P * ppr), qkv_weight,
                         out=dx[c * sc:(c + 1) * sc].view(sc * b, -1))
        return dx.view(T, -1), dq_full.view(T, P * ppr)
    finally:
        sched.end_region()


def _register_dense_dw(name: str, layer_id: int, x: torch.Tensor, dy: torch.Tensor, param,
                       transpose_out: bool = False) -> None:
    """Queue ``dW = dy^T @ x`` (``[N, K]``, the nn.Linear layout) or ``x^T @ dy`` when
    ``transpose_out`` (``[K, N]``)."""
    sched = get_backward_scheduler()

    def run():
        a, bm = (x, dy) if transpose_out else (dy, x)
        buf = sched._buffer_of(param) if sched.is_enabled() else None
        if buf is not None and param.main_grad.dtype == torch.float32 and a.is_cuda \
                and a.dtype == torch.bfloat16 and bm.shape[1] % 8 == 0 and a.shape[1] % 8 == 0:
            first = not getattr(param, "_ar_buf_written", False)
            gemm.grouped_gemm_wgrad(a, bm, 1, out=param.main_grad, accumulate=not first,
                                    max_ctas=sched.dw_max_ctas)
            return None
        return gemm.grouped_gemm_wgrad(a, bm, 1).view(param.shape)

    sched.register_dw_task(name, layer_id, run, param)


def register_qkv_dw(layer_id: int, ln1_out: torch.Tensor, dqkv_sp: torch.Tensor, qkv_param) -> None:
    """``dWqkv = dQKV^T @ ln1_out`` (fluid/attention/backward.py:399-421)."""
    _register_dense_dw("attn.qkv", layer_id, ln1_out, dqkv_sp, qkv_param)


def output_projection_register_dw(layer_id: int, attn_input_full: torch.Tensor, d_out: torch.Tensor,
                                  proj_param) -> None:
    """``dWproj = dOut^T @ attn_input_full`` (fluid/attention/backward.py:425-468)."""
    _register_dense_dw("attn.proj", layer_id, attn_input_full, d_out, proj_param)


def scaled_dot_product_attention_forward(q, k, v, scale=None, is_causal=True, enable_gqa=False):
    """``[b, h, s, d]`` inputs (the layout of the reference helper, fluid/attention/forward.py:280-329);
    returns ``[b, hq, s, d]``."""
    from ..ops import attention as attn_ops
    out, _ = attn_ops.attention_fwd(q.permute(2, 0, 1, 3), k.permute(2, 0, 1, 3), v.permute(2, 0, 1, 3),
                                    scale, is_causal)
    return out.permute(1, 2, 0, 3)


# names used by the reference for the same entry points
qkv_projection_p2p_forward = qkv_projection_forward
output_projection_p2p_forward = output_projection_forward
