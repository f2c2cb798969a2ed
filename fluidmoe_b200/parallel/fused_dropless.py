"""Dropless (variable-split) expert exchange on the device-initiated transport.

Every routed (token, expert) pair is kept, so the number of rows that travel between two ranks is
only known on the device.  Nothing here reads it back: the per-expert counts are exchanged with
peer stores, a one-CTA kernel turns the ``[P, E]`` table into row ranges (``group_rows`` /
``group_offs`` / arrival-counter bases of the local experts, destination rows of every run this
rank sends, the number of rows that come back from every rank), and the grouped GEMMs, the scatter
epilogues and the wait kernels take all of it from device memory
(``csrc/symm/dropless_kernels.cu``).  Receive buffers are sized for the worst case
``P * T * min(k, nle)`` rows (times ``buffer_factor`` when the caller knows the load is bounded);
a plan that does not fit is refused by every rank alike and reported through the status word.

The reference pads every expert to a fixed capacity and drops what does not fit
(fluid/moe/forward.py:387-417); its README-era API carried host-side ``input_splits /
output_splits`` (README:62-67).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native
from ..ops import gemm, permute
from ..ops.gemm import status_buffer


@dataclass
class DeviceDroplessPlan:
    """Sender-side routing of one forward pass; every field lives on the device."""
    sorted_indices: torch.Tensor     # [T*k] int64: token of every slot, slots sorted by global expert
    permuted_probs: torch.Tensor     # [T*k] fp32
    slot_of_token: torch.Tensor      # [T, k] int32: slot of the j-th choice of token t
    counts: torch.Tensor             # [E] int32 routed pairs per global expert
    routed_per_expert: torch.Tensor  # alias of counts (what the load-balancing loss reads)
    group_rows: Optional[torch.Tensor] = None   # [nle] rows per local expert (filled by the exchange)
    group_offs: Optional[torch.Tensor] = None   # [nle] first row of every local expert


def build_device_plan(top_idx: torch.Tensor, top_probs: torch.Tensor, num_experts: int) -> DeviceDroplessPlan:
    """Sort the (token, expert) pairs by expert, token order kept; no host synchronisation."""
    T, k = top_idx.shape
    dev = top_idx.device
    flat_e = top_idx.reshape(-1)
    order = torch.sort(flat_e, stable=True).indices
    sorted_indices = torch.div(order, k, rounding_mode="floor").to(torch.int64)
    permuted_probs = top_probs.reshape(-1).float()[order].contiguous()
    slot_of_token = torch.empty(T * k, dtype=torch.int32, device=dev)
    slot_of_token[order] = torch.arange(T * k, dtype=torch.int32, device=dev)
    counts = torch.zeros(num_experts, dtype=torch.int32, device=dev)
    counts.scatter_add_(0, flat_e.to(torch.int64), torch.ones_like(flat_e, dtype=torch.int32))
    return DeviceDroplessPlan(sorted_indices, permuted_probs, slot_of_token.view(T, k), counts, counts)


class _DroplessBuffers:
    def __init__(self, heap, ep_plan, dtype, buffer_factor: float):
        T, H, E, k = ep_plan.num_tokens, ep_plan.hidden_size, ep_plan.num_experts, ep_plan.top_k
        P, nle = ep_plan.ep_size, ep_plan.num_local_experts
        dev = heap.device
        worst = P * T * min(k, nle)
        rows = int(worst * min(1.0, max(buffer_factor, 0.0))) if buffer_factor else worst
        self.max_rows = ((max(rows, 128) + 127) // 128) * 128 + nle * 128
        self.slots = T * k
        self.tokens_em = heap.alloc((self.max_rows, H), dtype, zero=False)
        self.probs_em = heap.alloc((self.max_rows,), torch.float32)
        self.flags_fwd = heap.alloc((self.max_rows // 128,), torch.int32)
        self.dfc2_em = heap.alloc((self.max_rows, H), dtype, zero=False)
        self.flags_bwd = heap.alloc((self.max_rows // 128,), torch.int32)
        self.combined = heap.alloc((self.slots, H), dtype, zero=False)
        self.cnt_combine = heap.alloc((P,), torch.int32)
        self.dperm = heap.alloc((self.slots, H), dtype, zero=False)
        self.dprobs_perm = heap.alloc((self.slots,), torch.float32, zero=False)
        self.cnt_dperm = heap.alloc((P,), torch.int32)
        self.count_table = heap.alloc((2 * P * E,), torch.int32)
        self.count_flags = heap.alloc((P,), torch.int32)
        self.epoch = 0
        me = heap.rank
        self.cnt_combine_tbl = torch.tensor([a + 4 * me for a in self.cnt_combine.peer_addrs],
                                            dtype=torch.int64, device=dev)
        self.cnt_dperm_tbl = torch.tensor([a + 4 * me for a in self.cnt_dperm.peer_addrs],
                                          dtype=torch.int64, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        self.counts_all = torch.zeros(P * E, **i32)
        self.group_rows = torch.zeros(nle, **i32)
        self.group_offs = torch.zeros(nle, **i32)
        self.group_flag_base = torch.zeros(nle, **i32)
        self.dst_base = torch.zeros(E, **i32)
        self.slot_start = torch.zeros(E + 1, **i32)
        self.before = torch.zeros(P * nle, **i32)
        self.src_prefix = torch.zeros(P * E, **i32)
        self.recv_expected = torch.zeros(P, **i32)
        self.totals = torch.zeros(2, **i32)
        self.row_dst_rank = torch.full((self.max_rows,), -1, **i32)
        self.row_dst_row = torch.zeros(self.max_rows, **i32)
        self.plan_ptrs = [t.data_ptr() for t in (self.counts_all, self.group_rows, self.group_offs,
                                                 self.group_flag_base, self.dst_base, self.slot_start, self.before,
                                                 self.src_prefix, self.recv_expected, self.totals)]


class DroplessExchange:
    """The dropless forward and backward of one layer's expert block on a ``FusedCommContext``."""

    def __init__(self, ctx, buffer_factor: float = 0.0):
        self.ctx = ctx
        self.buffer_factor = buffer_factor      # 0: worst case

    # ------------------------------------------------------------------ helpers
    def _zero_padding(self, b: _DroplessBuffers, t: torch.Tensor) -> None:
        self.ctx_count()
        _native.lib().zero_group_padding(t.data_ptr(), t.stride(0) * t.element_size(), b.group_rows.data_ptr(),
                                         b.group_offs.data_ptr(), b.group_rows.numel(), _native.stream_ptr())

    def ctx_count(self, n: int = 1) -> None:
        from . import fused
        fused._count(n)

    def _gate(self, b: _DroplessBuffers, flags) -> dict:
        c = self.ctx
        return dict(gate_flags=flags.local.data_ptr(), gate_group_base=b.group_flag_base.data_ptr(),
                    gate_blocks_per_group=0, gate_expected=1, timeout_ns=c.timeout_ns, wait_ns=c._wait_ptr(0))

    def _dispatch(self, b, plan, ep, x, probs, dst_tokens, dst_probs, flags) -> None:
        c = self.ctx
        self.ctx_count()
        with c._Timed(c):
            _native.lib().dropless_dispatch(
                x.data_ptr(), plan.sorted_indices.data_ptr(), probs.data_ptr() if probs is not None else 0,
                b.plan_ptrs, dst_tokens.ptr_table, dst_probs.ptr_table if dst_probs is not None else 0,
                flags.ptr_table, b.slots, ep.hidden_size, ep.num_experts, ep.num_local_experts, ep.ep_size,
                ep.ep_rank, 0, _native.stream_ptr())

    def _scatter(self, b, ep, a, w, b_layout, dst, cnt_tbl, row_aux=None, row_aux_dst=None) -> None:
        """Grouped GEMM over the local experts' rows; the epilogue stores every row into the
        permuted-order buffer of the rank it came from."""
        c = self.ctx
        self.ctx_count()
        K = a.shape[1]
        N = w.shape[2] if b_layout == "kn" else w.shape[1]
        b2 = w.reshape(-1, w.shape[2])
        ap, ai, ao, lda = gemm._operand(a)
        bp, bi, bo, ldb = gemm._operand(b2)
        lib = _native.lib()
        desc = dict(
            A=ap, a_inner=ai, a_outer=ao, lda=lda, a_mn=0,
            B=bp, b_inner=bi, b_outer=bo, ldb=ldb, b_mn=1 if b_layout == "kn" else 0,
            mode=0, num_groups=w.shape[0], M=a.shape[0], N=N, K=K, b_group_stride=w.shape[1],
            uniform_rows=0, group_rows=b.group_rows.data_ptr(), group_offs=b.group_offs.data_ptr(),
            bn=256 if N > 128 else 128, epi=lib.EPI_SCATTER, dst_base=dst.ptr_table,
            dst_rank=b.row_dst_rank.data_ptr(), dst_row=b.row_dst_row.data_ptr(), ld_dst=ep.hidden_size,
            dst_flags=cnt_tbl.data_ptr(), num_ranks=ep.ep_size, timeout_ns=c.timeout_ns,
            status=status_buffer(a.device).data_ptr(), cta_pair=gemm.CTA_PAIR)
        if row_aux is not None:
            desc.update(row_aux=row_aux.data_ptr(), row_aux_dst=row_aux_dst.ptr_table)
        lib.gemm_launch(desc, _native.stream_ptr())

    # ------------------------------------------------------------------ forward
    def forward(self, b: _DroplessBuffers, ep, plan: DeviceDroplessPlan, x, w1, w2, activation, save_pre,
                needs_grad=None):
        """Returns ``(combined [T*k, H] in permuted order (complete only after ``wait_combined``),
        state for backward)``."""
        from ..models.moe import MoEForwardState
        from . import fused
        c = self.ctx
        lib = _native.lib()
        b.epoch += 1
        self.ctx_count(2)
        lib.dropless_plan(plan.counts.data_ptr(), b.count_table.ptr_table, b.count_flags.ptr_table, b.epoch,
                          ep.ep_size, ep.ep_rank, ep.num_experts, ep.num_local_experts,
                          c._n_tiles(ep.hidden_size) * fused.EPI_SPLIT, b.max_rows, b.plan_ptrs,
                          b.row_dst_rank.data_ptr(), b.row_dst_row.data_ptr(), c.timeout_ns,
                          status_buffer(c.device).data_ptr(), _native.stream_ptr())
        plan.group_rows, plan.group_offs = b.group_rows, b.group_offs
        self._zero_padding(b, b.tokens_em.local)
        self._dispatch(b, plan, ep, x, plan.permuted_probs, b.tokens_em, b.probs_em, b.flags_fwd)
        Fw = w1.shape[2]
        F = Fw // 2 if activation == "swiglu" else Fw
        act = torch.empty(b.max_rows, F, dtype=x.dtype, device=x.device)
        pre = torch.empty(b.max_rows, Fw, dtype=x.dtype, device=x.device) if save_pre else None
        gemm.grouped_gemm_act(b.tokens_em.local, w1, b.probs_em.local, activation=activation,
                              group_rows=b.group_rows, group_offs=b.group_offs, save_pre=save_pre,
                              gate=self._gate(b, b.flags_fwd), act_out=act, pre_out=pre)
        b.flags_fwd.local.zero_()
        if save_pre if needs_grad is None else needs_grad:
            # the weight-gradient GEMM reads whole 128-row groups: rows behind a group's last token
            # must be zero (they meet zero gradient rows, but uninitialised memory may hold NaN)
            self._zero_padding(b, act)
        self._scatter(b, ep, act, w2, "kn", b.combined, b.cnt_combine_tbl)
        return b.combined.local, MoEForwardState(b.tokens_em.local, b.probs_em.local, pre, act)

    def wait_rows(self, b: _DroplessBuffers, which: str) -> None:
        """Block the stream until every rank's rows are in ``combined`` / ``dperm``."""
        cnt = b.cnt_combine if which == "combined" else b.cnt_dperm
        self.ctx._wait_counters(cnt, 0, b.recv_expected)
        cnt.local.zero_()

    def unpermute(self, b, plan, rows, residual, which: str, waited: bool = False):
        if not waited:
            self.wait_rows(b, which)
        return permute.unpermute_reduce(rows, plan.slot_of_token, residual)

    # ------------------------------------------------------------------ backward
    def combine_fc2_backward(self, b, ep, plan, dy2, state, w2, activation):
        """Region moe_combine: output-gradient rows to the experts, FC2 input gradient and
        activation backward gated on their arrival.  Returns ``(dfc2_em, dpre_em, dprobs_em)``."""
        from .scheduler import get_backward_scheduler
        self._dispatch(b, plan, ep, dy2, None, b.dfc2_em, None, b.flags_bwd)
        self._zero_padding(b, b.dfc2_em.local)
        sched = get_backward_scheduler()
        if sched.is_enabled():
            sched.execute_dw_tasks(max_defer_tasks=2)
        dpre = torch.empty_like(state.pre_em)
        dpre, dprobs = gemm.grouped_gemm_dact(b.dfc2_em.local, w2, state.pre_em, state.probs_em,
                                              activation=activation, group_rows=b.group_rows,
                                              group_offs=b.group_offs, gate=self._gate(b, b.flags_bwd),
                                              dpre_out=dpre)
        b.flags_bwd.local.zero_()
        self._zero_padding(b, dpre)
        return b.dfc2_em.local, dpre, dprobs

    def fc1_dispatch_backward(self, b, ep, dpre_em, w1, dprobs_em):
        """Region moe_dispatch: FC1 input gradient whose epilogue returns every row, and the row's
        routing-probability gradient, to the token's owner."""
        from .scheduler import get_backward_scheduler
        self._scatter(b, ep, dpre_em, w1, "nk", b.dperm, b.cnt_dperm_tbl,
                      row_aux=dprobs_em.contiguous(), row_aux_dst=b.dprobs_perm)
        sched = get_backward_scheduler()
        if sched.is_enabled():
            sched.execute_dw_tasks(max_defer_tasks=2)
        return b.dperm.local
