"""Device-initiated expert-parallel exchange fused with the expert GEMMs.

For one expert-parallel group this context owns a symmetric heap and, per layer, the buffers the
peers write into:

* ``tokens_em`` / ``probs_em``: expert-major receive buffers of the dispatch.  The sender's
  permute kernel stores every routed row straight into the destination GPU's buffer and bumps the
  arrival counter of the row's 128-row block; the receiver's grouped FC1 GEMM (tcgen05) waits on
  that counter before its producer warp loads the block, so the first tiles start as soon as the
  local rows are in place and peer rows are consumed as they land.
* ``combined``: permuted-order buffer on the token owner.  The FC2 GEMM epilogue converts each
  accumulator row to bf16 and stores it into the owner's buffer over NVLink; per-source counters
  tell the owner when all rows of a source are in, then a gather-sum restores token order.
* the same two mechanisms, with the roles swapped, carry the backward pass (combine gradient in,
  dispatch gradient out).

Every wait is bounded and reports through the status word; counters are reset by their consumer
after use and a kernel-side barrier at the end of each iteration keeps iterations apart.

Buffer reuse.  The buffers are persistent per layer, so the same memory carries every iteration.
Three rules keep a write of iteration n+1 from landing on data of iteration n that is still needed:

1. *Exchange order.*  Every exchange is an all-to-all and every consumer kernel precedes, in its
   rank's stream, the next kernel that rank pushes with.  A rank reaches exchange k+1 only after its
   consumer of exchange k received the rows of every peer, i.e. after every peer launched its
   producer of exchange k, and that producer follows the peer's consumer of exchange k-1 in stream
   order.  So no rank can be more than one exchange ahead of another, and when a peer writes into a
   buffer of this rank for the second time, the kernel that read the first contents (and the
   ``zero_()`` of its counters, queued right behind it) has already been launched before the kernel
   whose output the peer waited for.  This holds for forward-only loops as well; no barrier is
   needed between forward passes.
2. *Deferred weight-gradient tasks* read ``tokens_em``, ``dfc2_em``, ``attn_in`` and ``dqkv_sp``
   after the backward pass that filled them.  ``layer_forward_begin`` therefore drains the
   scheduler's queue before a layer launches its first push of a new forward pass (gradient
   accumulation over micro-batches needs no barrier either).
3. *Tensors saved for backward* are views of these buffers.  A second forward pass of a layer
   before the backward pass of the first (two forwards then two backwards, or an evaluation pass
   in between) would overwrite them; ``layer_forward_begin`` raises instead.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist

from .. import _native
from ..ops import gemm, permute
from ..ops.gemm import status_buffer
from .symm import SymmetricHeap, SymmTensor

LAUNCHES = 0
EPI_SPLIT = 2   # epilogue warps per accumulator row (each reports its half of the columns)


def _count(n=1):
    global LAUNCHES
    LAUNCHES += n


class _LayerBuffers:
    def __init__(self, heap: SymmetricHeap, plan, dtype, ffn_cols: int):
        R, H = plan.rows_local, plan.hidden_size
        P, nle, cap = plan.ep_size, plan.num_local_experts, plan.expert_capacity
        self.bpg = (P * cap + 127) // 128                      # 128-row blocks per local expert
        nblk = nle * self.bpg
        dev = heap.device
        self.tokens_em = heap.alloc((R, H), dtype, zero=False)
        self.probs_em = heap.alloc((R,), torch.float32)
        self.flags_fwd = heap.alloc((nblk,), torch.int32)
        self.dfc2_em = heap.alloc((R, H), dtype, zero=False)
        self.flags_bwd = heap.alloc((nblk,), torch.int32)
        self.combined = heap.alloc((P * plan.S, H), dtype, zero=False)
        self.cnt_combine = heap.alloc((P,), torch.int32)
        self.dperm = heap.alloc((P * plan.S, H), dtype, zero=False)
        self.dprobs_perm = heap.alloc((P * plan.S,), torch.float32, zero=False)   # rides with dperm rows
        self.cnt_dperm = heap.alloc((P,), torch.int32)
        me = heap.rank
        # entry p = address of rank p's counter for rows coming from this rank
        self.cnt_combine_tbl = torch.tensor([a + 4 * me for a in self.cnt_combine.peer_addrs],
                                            dtype=torch.int64, device=dev)
        self.cnt_dperm_tbl = torch.tensor([a + 4 * me for a in self.cnt_dperm.peer_addrs],
                                          dtype=torch.int64, device=dev)


class _AttnBuffers:
    """Symmetric buffers of the Ulysses exchanges of one layer."""

    def __init__(self, heap: SymmetricHeap, cp, dtype):
        P, sl, b = cp.cp_size, cp.seq_local, cp.batch
        T = sl * b
        self.row_blocks = (T + 127) // 128
        dev = heap.device
        me = heap.rank
        self.qkv_full = heap.alloc((P * T, cp.proj_per_rank), dtype, zero=False)       # [s_full*b, ppr]
        self.cnt_qkv = heap.alloc((P,), torch.int32)
        self.attn_in = heap.alloc((T, P * cp.attn_per_rank), dtype, zero=False)        # [T, n_h*d]
        self.flags_proj = heap.alloc((P * self.row_blocks,), torch.int32)
        self.d_attn = heap.alloc((P * T, cp.attn_per_rank), dtype, zero=False)         # [s_full*b, dpr]
        self.cnt_dattn = heap.alloc((P,), torch.int32)
        self.dqkv_sp = heap.alloc((T, P * cp.proj_per_rank), dtype, zero=False)        # [T, P*ppr]
        self.flags_dqkv = heap.alloc((P * self.row_blocks,), torch.int32)
        self.cnt_qkv_tbl = torch.tensor([a + 4 * me for a in self.cnt_qkv.peer_addrs], dtype=torch.int64, device=dev)
        self.cnt_dattn_tbl = torch.tensor([a + 4 * me for a in self.cnt_dattn.peer_addrs], dtype=torch.int64, device=dev)


class FusedCommContext:
    supports_attention = True

    def __init__(self, group, heap_bytes: int, device, timeout_ms: float = 8000.0):
        self.group = group
        self.device = torch.device(device)
        self.heap = SymmetricHeap(group, heap_bytes, self.device)
        self.rank, self.world = self.heap.rank, self.heap.world
        self.timeout_ns = int(timeout_ms * 1e6)
        self._pending_wait = None
        self._layers: Dict[int, _LayerBuffers] = {}
        self._attn: Dict[int, _AttnBuffers] = {}
        self._sig: Dict[int, tuple] = {}
        self._awaiting_backward: Dict[int, bool] = {}
        self.generation = 0          # bumped whenever every buffer is released (a new input shape)
        from .fused_dropless import DroplessExchange
        self.dropless = DroplessExchange(self)
        # exposed-communication accounting (off by default): [0] ns producers of gated GEMMs waited
        # for rows (summed over CTAs), [1] ns the stand-alone wait kernels waited
        self._wait_ns = torch.zeros(2, dtype=torch.int64, device=self.device)
        self.metrics_enabled = False
        self._push_events: list = []
        self._gated_ctas = 0
        self.heap.mark()

    @staticmethod
    def attention_supported(cp_plan) -> bool:
        """The fused Ulysses paths move whole 64-column blocks per source."""
        return cp_plan is None or (cp_plan.proj_per_rank % 64 == 0 and cp_plan.attn_per_rank % 64 == 0)

    # ------------------------------------------------------------------ set-up
    def prepare(self, ep_plan, cp_plan, layer) -> None:
        """Allocate (first call) or re-allocate (new input shape) the buffers of ``layer``.  The heap
        is a bump allocator, so a new shape releases the buffers of every layer; each layer notices
        through ``generation`` and allocates again at its next forward pass.  Collective: every rank
        of the group must see the same shapes in the same order."""
        key = id(layer)
        sig = (ep_plan.signature(), cp_plan.signature() if cp_plan is not None else None)
        if self._sig.get(key) == sig and key in self._layers:
            return
        if key in self._layers:
            self._release_all()
        self._sig[key] = sig
        if getattr(layer, "dropless", False):
            # variable-split routing: worst-case sized receive buffers and the device-side plan
            from .fused_dropless import _DroplessBuffers
            self._layers[key] = _DroplessBuffers(self.heap, ep_plan, ep_plan.dtype, self.dropless.buffer_factor)
        else:
            self._layers[key] = _LayerBuffers(self.heap, ep_plan, ep_plan.dtype, layer.ffn_hidden_size)
        ep_plan._fused_layer = key
        if cp_plan is not None and cp_plan.cp_size > 1 and self.attention_supported(cp_plan):
            self._attn[key] = _AttnBuffers(self.heap, cp_plan, cp_plan.dtype)
            cp_plan._fused_layer = key
        self._awaiting_backward[key] = False
        # every rank must finish allocating (and zeroing counters) before anyone pushes
        self.heap.sync_group()

    def release_all(self) -> None:
        """Give every layer's buffers back to the heap (collective).  Layers that are used again
        allocate anew at their next forward pass."""
        if self._layers:
            self._release_all()

    def _release_all(self) -> None:
        if any(self._awaiting_backward.values()):
            raise RuntimeError("input shape changed between the forward and the backward pass of a layer")
        self.heap.sync_group()          # nobody is still reading or writing the old buffers
        self._layers.clear()
        self._attn.clear()
        self._sig.clear()
        self._awaiting_backward.clear()
        self.heap.release_to_mark()
        self.heap.mark()
        self.generation += 1

    def layer_forward_begin(self, ep_plan, needs_grad: bool) -> None:
        """First thing a layer does in a forward pass that uses these buffers (rules 2 and 3 of the
        module docstring)."""
        key = ep_plan._fused_layer
        if self._awaiting_backward.get(key, False):
            raise RuntimeError(
                "fused transport: this layer ran a forward pass whose backward pass has not run yet; its "
                "saved activations live in per-layer symmetric buffers that a second forward pass would "
                "overwrite. Run forward and backward alternately (gradient accumulation does), or use "
                "comm_mode='p2p' / 'a2a' for this pattern.")
        from .scheduler import get_backward_scheduler
        sched = get_backward_scheduler()
        if sched.is_enabled() and sched.num_queued_dw_tasks() > 0:
            sched.execute_dw_tasks()
        if sched.is_enabled():
            sched.join_dw_stream()      # side-stream tasks read this layer's buffers too
        self._awaiting_backward[key] = bool(needs_grad)

    def layer_backward_end(self, ep_plan) -> None:
        self._awaiting_backward[ep_plan._fused_layer] = False

    # ------------------------------------------------------------------ exposed-communication metrics
    def enable_comm_metrics(self, enabled: bool = True) -> None:
        """Count, from now on, the communication time the compute stream could not hide: time the
        producers of the gated GEMMs waited for rows, time the stand-alone wait kernels waited and
        the run time of the push kernels (measured with events)."""
        self.metrics_enabled = bool(enabled)
        self.reset_comm_metrics()

    def reset_comm_metrics(self) -> None:
        self._wait_ns.zero_()
        self._push_events.clear()
        self._gated_launches = 0

    def comm_metrics(self, num_ctas: int = 148) -> dict:
        """Milliseconds since the last reset (synchronises the device).  ``gated_gemm_wait`` is the
        per-CTA average of the producers' waits, an upper bound of what the tensor cores lost
        (the shared-memory ring keeps them fed for a few blocks while a producer waits)."""
        torch.cuda.synchronize(self.device)
        w = self._wait_ns.tolist()
        push = sum(s.elapsed_time(e) for s, e in self._push_events)
        out = dict(gated_gemm_wait_ms=w[0] / 1e6 / max(1, num_ctas), wait_kernels_ms=w[1] / 1e6, push_kernels_ms=push)
        out["exposed_comm_ms"] = out["gated_gemm_wait_ms"] + out["wait_kernels_ms"] + out["push_kernels_ms"]
        return out

    def _wait_ptr(self, slot: int) -> int:
        return self._wait_ns.data_ptr() + 8 * slot if self.metrics_enabled else 0

    class _Timed:
        def __init__(self, ctx):
            self.ctx = ctx

        def __enter__(self):
            if self.ctx.metrics_enabled:
                self.s = torch.cuda.Event(enable_timing=True)
                self.s.record()

        def __exit__(self, *exc):
            if self.ctx.metrics_enabled:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                self.ctx._push_events.append((self.s, e))

    def _buf(self, plan) -> _LayerBuffers:
        return self._layers[plan._fused_layer]

    def iteration_barrier(self) -> None:
        """Kernel-side barrier over the group; call once per iteration after the backward pass."""
        _count()
        self.heap.barrier(self.timeout_ns / 1e6)

    # ------------------------------------------------------------------ primitives
    def _push(self, plan, x, sorted_indices, probs, dst_tokens: SymmTensor, dst_probs: Optional[SymmTensor],
              flags: SymmTensor, bpg: int) -> None:
        _count()
        with self._Timed(self):
            _native.lib().permute_dispatch(
                x.data_ptr(), sorted_indices.data_ptr(), probs.data_ptr() if probs is not None else 0,
                dst_tokens.ptr_table, dst_probs.ptr_table if dst_probs is not None else 0, flags.ptr_table,
                plan.num_experts * plan.expert_capacity, plan.hidden_size, plan.expert_capacity,
                plan.num_local_experts, plan.ep_size, plan.ep_rank, bpg, 0, _native.stream_ptr())

    def _gate(self, flags: SymmTensor, bpg: int) -> dict:
        return dict(gate_flags=flags.local.data_ptr(), gate_blocks_per_group=bpg, gate_expected=1,
                    timeout_ns=self.timeout_ns, wait_ns=self._wait_ptr(0))

    def _scatter_gemm(self, plan, a, w, b_layout, dst: SymmTensor, cnt_tbl: torch.Tensor,
                      row_aux: Optional[torch.Tensor] = None, row_aux_dst: Optional[SymmTensor] = None) -> None:
        """Grouped GEMM over the expert-major rows whose epilogue stores each result row into the
        owner's buffer (``plan.combine_dst_rank`` / ``combine_dst_row``).  ``row_aux`` (fp32, one
        value per source row) travels with its row into ``row_aux_dst`` at the same destination
        row and is published by the same counter."""
        _count()
        G = w.shape[0]
        K = a.shape[1]
        N = w.shape[2] if b_layout == "kn" else w.shape[1]
        b2 = w.reshape(-1, w.shape[2])
        ap, ai, ao, lda = gemm._operand(a)
        bp, bi, bo, ldb = gemm._operand(b2)
        lib = _native.lib()
        desc = dict(
            A=ap, a_inner=ai, a_outer=ao, lda=lda, a_mn=0,
            B=bp, b_inner=bi, b_outer=bo, ldb=ldb, b_mn=1 if b_layout == "kn" else 0,
            mode=0, num_groups=G, M=a.shape[0], N=N, K=K, b_group_stride=w.shape[1],
            uniform_rows=plan.ep_size * plan.expert_capacity, bn=256 if N > 128 else 128,
            epi=lib.EPI_SCATTER, dst_base=dst.ptr_table, dst_rank=plan.combine_dst_rank.data_ptr(),
            dst_row=plan.combine_dst_row.data_ptr(), ld_dst=plan.hidden_size,
            dst_flags=cnt_tbl.data_ptr(), num_ranks=plan.ep_size,
            timeout_ns=self.timeout_ns, status=status_buffer(a.device).data_ptr(), cta_pair=gemm.CTA_PAIR)
        if row_aux is not None:
            assert row_aux.dtype == torch.float32 and row_aux.is_contiguous() and row_aux.numel() == a.shape[0]
            desc.update(row_aux=row_aux.data_ptr(), row_aux_dst=row_aux_dst.ptr_table)
        lib.gemm_launch(desc, _native.stream_ptr())

    def _wait_counters(self, cnt: SymmTensor, expected: int, expected_dev: Optional[torch.Tensor] = None) -> None:
        """Stand-alone wait for per-source arrival counters: ``expected`` for every source, or the
        per-source values of ``expected_dev`` (int32 on the device)."""
        _count()
        _native.lib().a2a_wait_counts(cnt.local.data_ptr(), self.world, expected,
                                      expected_dev.data_ptr() if expected_dev is not None else 0,
                                      self._wait_ptr(1), self.timeout_ns,
                                      status_buffer(self.device).data_ptr(), _native.stream_ptr())

    @staticmethod
    def _n_tiles(n: int) -> int:
        bn = 256 if n > 128 else 128
        return (n + bn - 1) // bn

    # ------------------------------------------------------------------ forward
    def dispatch_fc1(self, plan, hidden_states, sorted_indices, probs32, w1, activation, save_pre):
        from ..models.moe import MoEForwardState
        b = self._buf(plan)
        self._push(plan, hidden_states, sorted_indices, probs32, b.tokens_em, b.probs_em, b.flags_fwd, b.bpg)
        act, pre = gemm.grouped_gemm_act(b.tokens_em.local, w1, b.probs_em.local, activation=activation,
                                         uniform_rows=plan.ep_size * plan.expert_capacity,
                                         save_pre=save_pre, gate=self._gate(b.flags_fwd, b.bpg))
        b.flags_fwd.local.zero_()
        return MoEForwardState(b.tokens_em.local, b.probs_em.local, pre, act)

    def fc2_combine(self, plan, state, w2):
        b = self._buf(plan)
        self._scatter_gemm(plan, state.act_em, w2, "kn", b.combined, b.cnt_combine_tbl)
        return b.combined.local

    def unpermute(self, plan, rows, slot_of_token, residual, waited: bool = False):
        """Wait until every source's rows are in ``rows`` (the combine or dispatch-gradient buffer
        of this layer), then gather-sum them into token order.  ``waited``: the caller has already
        waited for (and reset) the counters with ``wait_dispatch_grad``."""
        b = self._buf(plan)
        cnt = b.cnt_combine if rows.data_ptr() == b.combined.local.data_ptr() else b.cnt_dperm
        out = None
        if not waited:
            # the gather kernel polls the arrival counters itself; a stand-alone wait kernel only when
            # the native gather cannot take this input
            expected = plan.S * self._n_tiles(plan.hidden_size) * EPI_SPLIT
            out = permute.unpermute_reduce(rows, slot_of_token, residual, wait=dict(
                flags=cnt.local.data_ptr(), n=self.world, expected=expected, wait_ns=self._wait_ptr(1),
                timeout_ns=self.timeout_ns, status=status_buffer(self.device).data_ptr()))
            if out is None:
                self._wait_counters(cnt, expected)
        if out is None:
            out = permute.unpermute_reduce(rows, slot_of_token, residual)
        if not waited:
            cnt.local.zero_()
        return out

    # ------------------------------------------------------------------ backward
    def combine_fc2_backward(self, plan, dy2, rplan, state, w2, activation):
        from .scheduler import get_backward_scheduler
        b = self._buf(plan)
        sched = get_backward_scheduler()
        self._push(plan, dy2, rplan.sorted_indices, None, b.dfc2_em, None, b.flags_bwd, b.bpg)
        if sched.is_enabled():
            sched.execute_dw_tasks(max_defer_tasks=2)
        dpre, dprobs = gemm.grouped_gemm_dact(b.dfc2_em.local, w2, state.pre_em, state.probs_em,
                                              activation=activation,
                                              uniform_rows=plan.ep_size * plan.expert_capacity,
                                              gate=self._gate(b.flags_bwd, b.bpg))
        b.flags_bwd.local.zero_()
        return b.dfc2_em.local, dpre, dprobs

    def fc1_dispatch_backward(self, plan, dpre_em, w1, dprobs_em=None):
        """Region moe_dispatch: ``dTok = dpre @ W1^T`` whose epilogue stores every row into the
        token owner's ``dperm`` buffer; with ``dprobs_em`` the routing-probability gradient of the
        row goes with it (the reference sends it through a separate synchronous all-to-all,
        fluid/layer/transformer.py:526-538)."""
        from .scheduler import get_backward_scheduler
        b = self._buf(plan)
        self._scatter_gemm(plan, dpre_em, w1, "nk", b.dperm, b.cnt_dperm_tbl,
                           row_aux=dprobs_em, row_aux_dst=b.dprobs_perm if dprobs_em is not None else None)
        sched = get_backward_scheduler()
        if sched.is_enabled():
            sched.execute_dw_tasks(max_defer_tasks=2)
        return b.dperm.local

    def wait_dispatch_grad(self, plan) -> torch.Tensor:
        """Block the stream until every source's dispatch-gradient rows (and the probability
        gradients that came with them) are in; returns the probability gradients in permuted order."""
        b = self._buf(plan)
        self._wait_counters(b.cnt_dperm, plan.S * self._n_tiles(plan.hidden_size) * EPI_SPLIT)
        b.cnt_dperm.local.zero_()
        return b.dprobs_perm.local


    # ------------------------------------------------------------------ Ulysses exchanges
    def _colscatter_gemm(self, a, w, b_layout, P, cols_per_rank, dst: SymmTensor, cnt_tbl, row_offset):
        """``a @ W`` whose column block p is stored into rank p's buffer at row ``row_offset + row``.
        N tiles are visited starting right after this rank's own block, so remote data leaves first
        and the local block is written last."""
        _count()
        K = a.shape[1]
        N = w.shape[1] if b_layout == "kn" else w.shape[0]
        ap, ai, ao, lda = gemm._operand(a)
        bp, bi, bo, ldb = gemm._operand(w)
        lib = _native.lib()
        bn = 256 if N > 128 else 128
        nt = (N + bn - 1) // bn
        me = self.rank
        rot = (((me + 1) % P) * cols_per_rank // bn) % nt if cols_per_rank % bn == 0 else 0
        desc = dict(
            A=ap, a_inner=ai, a_outer=ao, lda=lda, a_mn=0,
            B=bp, b_inner=bi, b_outer=bo, ldb=ldb, b_mn=1 if b_layout == "kn" else 0,
            mode=0, num_groups=1, M=a.shape[0], N=N, K=K, b_group_stride=0, uniform_rows=a.shape[0],
            bn=bn, epi=lib.EPI_COLSCATTER, dst_base=dst.ptr_table, ld_dst=cols_per_rank,
            cols_per_rank=cols_per_rank, dst_row_offset=row_offset, dst_flags=cnt_tbl.data_ptr(),
            num_ranks=P, n_rotate=rot, timeout_ns=self.timeout_ns,
            status=status_buffer(a.device).data_ptr(), cta_pair=gemm.CTA_PAIR)
        lib.gemm_launch(desc, _native.stream_ptr())

    def _rows_push(self, src2d, P, dst: SymmTensor, flags: SymmTensor, row_blocks):
        _count()
        rows_blk = src2d.shape[0] // P
        with self._Timed(self):
            _native.lib().rows_push(src2d.data_ptr(), dst.ptr_table, flags.ptr_table, rows_blk, src2d.shape[1],
                                    P, self.rank, row_blocks, 0, _native.stream_ptr())

    def _ksource_gate(self, flags: SymmTensor, cols_per_src: int, row_blocks: int, units_per_row: int = 1) -> dict:
        return dict(gate_flags=flags.local.data_ptr(), gate_k_blocks_per_src=cols_per_src // 64,
                    gate_blocks_per_group=row_blocks, k_rotate=self.rank * (cols_per_src // 64),
                    gate_expected=units_per_row, timeout_ns=self.timeout_ns, wait_ns=self._wait_ptr(0))

    def attention_push_args(self, plan, qkv_full):
        """Arguments that let the attention kernel do the HP -> SP exchange in its epilogue, or
        ``None`` when it cannot (batch > 1, rows per rank not a multiple of 128, other kernel)."""
        from ..ops import attention as attn_ops, flash
        T = plan.seq_local * plan.batch
        if not attn_ops.native_forward(qkv_full, plan.head_dim) or not flash.can_push(qkv_full, T):
            return None
        b = self._attn[plan._fused_layer]
        return dict(dst_table=b.attn_in.ptr_table, flags_table=b.flags_proj.ptr_table, me=self.rank,
                    P=plan.cp_size, rows_per_rank=T, row_blocks=b.row_blocks)

    # ---- waits handed to the first consumer kernel instead of a stand-alone wait kernel ----
    def _wait_or_defer(self, cnt: SymmTensor, expected: int, defer: bool) -> None:
        if defer:
            assert self._pending_wait is None, "the previous deferred wait was never consumed"
            self._pending_wait = (cnt, expected)
        else:
            self._wait_counters(cnt, expected)
            cnt.local.zero_()

    def take_pending_wait(self):
        """Arguments for the kernel that reads the buffer peers are still filling (it waits for the
        arrival counters in its prologue); ``standalone`` runs the stand-alone wait kernel for
        back-ends that cannot.  The caller ends with ``finish_pending_wait()``."""
        cnt, expected = self._pending_wait
        return dict(flags=cnt.local.data_ptr(), n=self.world, expected=expected, wait_ns=self._wait_ptr(1),
                    timeout_ns=self.timeout_ns, status=status_buffer(self.device).data_ptr(),
                    standalone=lambda: self._wait_counters(cnt, expected))

    def finish_pending_wait(self) -> None:
        cnt, _ = self._pending_wait
        self._pending_wait = None
        cnt.local.zero_()

    def qkv_sp2hp(self, x, qkv_weight, plan, defer_wait: bool = False):
        """QKV projection whose epilogue performs the SP->HP exchange (fluid/attention/forward.py:130-277).
        ``defer_wait``: the caller's next kernel (RoPE) waits for the peers' column blocks itself."""
        b = self._attn[plan._fused_layer]
        P, sl, bt, ppr = plan.cp_size, plan.seq_local, plan.batch, plan.proj_per_rank
        T = sl * bt
        self._colscatter_gemm(x, qkv_weight, "nk", P, ppr, b.qkv_full, b.cnt_qkv_tbl, self.rank * T)
        self._wait_or_defer(b.cnt_qkv, T * (ppr // 32), defer_wait)
        return b.qkv_full.local.view(P * sl, bt, plan.groups_per_rank, plan.group_size)

    def hp2sp_outproj(self, attn_out, proj_weight, plan, residual, pushed: bool = False):
        """HP->SP push followed by the output projection whose K loop consumes each source's
        column block as it arrives, local block first (fluid/attention/forward.py:332-484).
        ``pushed``: the attention kernel's epilogue has already stored the rows at their owners
        (one arrival per row and head), so there is nothing left to push."""
        b = self._attn[plan._fused_layer]
        P, sl, bt, dpr = plan.cp_size, plan.seq_local, plan.batch, plan.attn_per_rank
        T = sl * bt
        if not pushed:
            self._rows_push(attn_out.reshape(P * T, dpr), P, b.attn_in, b.flags_proj, b.row_blocks)
        out = residual.clone() if residual is not None else None
        out = gemm.grouped_gemm(b.attn_in.local, proj_weight, b_layout="nk", out=out,
                                accumulate=residual is not None,
                                gate=self._ksource_gate(b.flags_proj, dpr, b.row_blocks,
                                                        plan.heads_per_rank if pushed else 1))
        b.flags_proj.local.zero_()
        return out, b.attn_in.local

    def outproj_dx_sp2hp(self, d_out, proj_weight, plan, defer_wait: bool = False):
        """Region attn_proj: ``dAttn = dOut @ Wproj`` with the SP->HP exchange in the epilogue.
        ``defer_wait``: the attention backward's first kernel waits for the peers' blocks itself."""
        from .scheduler import get_backward_scheduler
        b = self._attn[plan._fused_layer]
        P, sl, bt, dpr = plan.cp_size, plan.seq_local, plan.batch, plan.attn_per_rank
        T = sl * bt
        self._colscatter_gemm(d_out, proj_weight, "kn", P, dpr, b.d_attn, b.cnt_dattn_tbl, self.rank * T)
        sched = get_backward_scheduler()
        if sched.is_enabled():
            sched.execute_dw_tasks(max_defer_tasks=2)
        self._wait_or_defer(b.cnt_dattn, T * (dpr // 32), defer_wait)
        return b.d_attn.local.view(P * sl, bt, plan.heads_per_rank, plan.head_dim)

    def hp2sp_qkv_dx(self, dqkv_hp, qkv_weight, plan):
        """Region attn_qkv: HP->SP push of dQKV, then ``dX = dQKV @ Wqkv`` gated along K by source."""
        from .scheduler import get_backward_scheduler
        b = self._attn[plan._fused_layer]
        P, sl, bt, ppr = plan.cp_size, plan.seq_local, plan.batch, plan.proj_per_rank
        T = sl * bt
        self._rows_push(dqkv_hp.reshape(P * T, ppr), P, b.dqkv_sp, b.flags_dqkv, b.row_blocks)
        sched = get_backward_scheduler()
        if sched.is_enabled():
            sched.execute_dw_tasks(max_defer_tasks=2)
        dx = gemm.grouped_gemm(b.dqkv_sp.local, qkv_weight, b_layout="kn",
                               gate=self._ksource_gate(b.flags_dqkv, ppr, b.row_blocks))
        b.flags_dqkv.local.zero_()
        return dx, b.dqkv_sp.local
