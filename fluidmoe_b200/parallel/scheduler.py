"""Backward scheduler: deferred weight-gradient work, asynchronous all-to-alls, trickled all-reduce.

Responsibilities (same contract as the reference's BackwardScheduler, fluid/core/scheduler.py):

* a FIFO of weight-gradient tasks that the backward pass registers instead of computing; a bounded
  number of them is executed inside each communication window (``execute_dw_tasks``) and the rest
  flows on to the windows of earlier layers or to ``finish_batch``;
* submission of all-to-alls on the communication stream with pooled hand-off events, and
  ``wait_alltoall`` on the compute stream;
* flat gradient buffers with write / committed / read cursors, whose committed prefix is
  all-reduced in slices sized by a per-region time budget whenever no all-to-all is outstanding;
* three modes: F (disabled: everything synchronous), FB (deferred dW, one all-reduce at the
  end), full (deferred dW + trickled all-reduce);
* region profiles, gap profiles and exposed-communication metrics.

Decisions never depend on GPU timing, so every rank issues collectives in the same order.
On CPU tensors streams and events degrade to no-ops and the same code runs synchronously.
"""
from __future__ import annotations

import collections
import contextlib
import os
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.overhead_profiler import get_overhead_profiler
from .streams import NullStream, current_stream, get_stream_manager, make_event, on_stream

BACKWARD_REGIONS = ("moe_combine", "moe_dispatch", "attn_proj", "attn_qkv")
FORWARD_REGIONS = ("r1_f", "r2_f", "r3_f", "r4_f")


@dataclass
class DWTask:
    layer_name: str
    layer_id: int
    compute_fn: Callable[[], Optional[torch.Tensor]]
    weight_param: Optional[torch.nn.Parameter] = None
    needs_ar: bool = True
    target_buffer: Optional[torch.Tensor] = None
    defer: bool = True


class FlatGradBuffer:
    """Contiguous gradient storage for a list of parameters, reduced front to back.

    Parameters are laid out in the order given (callers pass them in backward order, so the
    prefix that is complete first is also the first to be reduced).  ``write`` marks how far
    gradients have been produced, ``committed`` how far they are final for this iteration, and
    ``read`` how far they have been handed to the all-reduce.
    Counterpart of fluid/core/scheduler.py:35-216.
    """

    def __init__(self):
        self.buffers: Dict[torch.dtype, torch.Tensor] = {}
        self.param_map: Dict[int, tuple] = {}   # id(param) -> (dtype, offset, numel)
        self.order: List[torch.nn.Parameter] = []
        self.write = 0      # elements, per primary buffer
        self.committed = 0
        self.read = 0
        self.primary: Optional[torch.dtype] = None
        self._written_upto: Dict[torch.dtype, int] = {}

    def setup(self, params, accumulate_in_fp32: bool = False, allocator=None) -> None:
        params = [p for p in params if p is not None]
        self.order = params
        sizes: Dict[torch.dtype, int] = collections.OrderedDict()
        self.param_map.clear()
        for p in params:
            dt = torch.float32 if accumulate_in_fp32 else p.dtype
            off = sizes.get(dt, 0)
            self.param_map[id(p)] = (dt, off, p.numel())
            sizes[dt] = off + p.numel()
        self.buffers = {}
        for dt, n in sizes.items():
            dev = params[0].device
            self.buffers[dt] = (allocator(n, dt) if allocator else
                                torch.zeros(n, dtype=dt, device=dev))
        self.primary = next(iter(sizes)) if sizes else None
        for p in params:
            dt, off, n = self.param_map[id(p)]
            p.main_grad = self.buffers[dt][off:off + n].view(p.shape)
            p._ar_buf_written = False
        self.reset_cursors()

    def __contains__(self, param) -> bool:
        return id(param) in self.param_map

    @property
    def numel(self) -> int:
        return sum(b.numel() for b in self.buffers.values())

    def reset_cursors(self) -> None:
        self.write = self.committed = self.read = 0
        self._written_upto = {dt: 0 for dt in self.buffers}
        self._done = set()
        self._next = 0   # index into ``order`` of the first primary-dtype parameter not yet written

    def zero(self) -> None:
        for b in self.buffers.values():
            b.zero_()
        for p in self.order:
            p._ar_buf_written = False
        self.reset_cursors()

    def write_grad(self, param, grad: Optional[torch.Tensor]) -> None:
        """First write of an iteration copies, later writes accumulate.  ``grad`` may be None
        when the producing kernel already accumulated into ``param.main_grad`` in place."""
        dt, off, n = self.param_map[id(param)]
        view = self.buffers[dt][off:off + n]
        if grad is not None:
            g = grad.reshape(-1)
            if getattr(param, "_ar_buf_written", False):
                view.add_(g)
            else:
                view.copy_(g)
        param._ar_buf_written = True
        self._written_upto[dt] = max(self._written_upto[dt], off + n)
        self._done.add(id(param))
        # ``write`` only moves over a prefix whose parameters have all been produced, so a
        # gradient that arrives out of layout order can never be skipped by the all-reduce.
        while self._next < len(self.order):
            nxt = self.order[self._next]
            ndt, noff, nn_ = self.param_map[id(nxt)]
            if ndt != self.primary:
                self._next += 1
                continue
            if id(nxt) not in self._done:
                break
            self.write = noff + nn_
            self._next += 1

    def commit(self) -> None:
        self.committed = self.write

    def commit_all(self) -> None:
        """End of the backward pass: everything in the buffer is final."""
        if self.primary is not None:
            self.write = self.committed = self.buffers[self.primary].numel()

    def has_pending(self) -> bool:
        return self.read < self.committed

    def has_remainder(self) -> bool:
        """True while anything written, committed or not, is still unreduced
        (fluid/core/scheduler.py:112-115)."""
        return self.read < self.write

    def pending_bytes(self) -> int:
        if self.primary is None:
            return 0
        return (self.committed - self.read) * self.buffers[self.primary].element_size()

    def submit_block(self, reduce_fn: Callable[[torch.Tensor, float], None], max_bytes: int = 0,
                     pre_scale: float = 1.0, ceiling: Optional[int] = None) -> int:
        """Reduce ``[read, min(committed, ceiling))`` (at most ``max_bytes`` when > 0)."""
        if self.primary is None:
            return 0
        buf = self.buffers[self.primary]
        hi = self.committed if ceiling is None else min(self.committed, ceiling)
        n = hi - self.read
        if n <= 0:
            return 0
        if max_bytes > 0:
            n = min(n, max(1, max_bytes // buf.element_size()))
        chunk = buf[self.read:self.read + n]
        reduce_fn(chunk, pre_scale)
        self.read += n
        return n * buf.element_size()

    def sync_allreduce(self, reduce_fn, pre_scale: float = 1.0) -> int:
        total = 0
        for dt, buf in self.buffers.items():
            if dt == self.primary:
                lo = self.read
                if lo < buf.numel():
                    reduce_fn(buf[lo:], pre_scale)
                    total += (buf.numel() - lo) * buf.element_size()
                self.read = self.committed = self.write = buf.numel()
            else:
                reduce_fn(buf, pre_scale)
                total += buf.numel() * buf.element_size()
        return total

    def skip_pending(self) -> None:
        """Nothing in this buffer needs a reduction (its gradients were consumed in place)."""
        if self.primary is not None:
            self.read = self.committed

    def consumed_in_backward(self) -> bool:
        """True when every parameter of the buffer is updated by its weight-gradient GEMM."""
        return bool(self.order) and all(getattr(p, "_fused_adam", None) is not None for p in self.order)

    def scale_pending(self, scale: float) -> None:
        for buf in self.buffers.values():
            buf.mul_(scale)


_FlatARBuffer = FlatGradBuffer


def _default_reduce(group):
    def fn(chunk: torch.Tensor, pre_scale: float):
        if pre_scale != 1.0:
            chunk.mul_(pre_scale)
        if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(chunk, group=group)
    return fn


class BackwardScheduler:
    _instance: Optional["BackwardScheduler"] = None

    def __new__(cls):
        if cls._instance is None:
            inst = super().__new__(cls)
            inst._init_state()
            cls._instance = inst
        return cls._instance

    # ------------------------------------------------------------------ state
    def _init_state(self) -> None:
        self.enabled = False
        self.ar_enabled = False
        # ablation switches
        self.stage2_enabled = True        # run dW tasks inside communication windows
        # Ablations under the reference's environment names (fluid/moe/backward.py:40-41,280-287):
        # keep deferrable dW tasks out of every window / out of the dispatch-gradient window only.
        self.skip_all_dw = os.environ.get("FLUID_SKIP_ALL_DW", "0") == "1"
        self.skip_dispatch_dw = os.environ.get("FLUID_SKIP_DISPATCH_DW", "0") == "1"
        self.cross_region_flow = True     # leftovers flow into later windows
        self.use_profiled_gaps = True
        self.fixed_ar_budget = 0          # bytes per gap when > 0 (overrides the model)
        self.pending_ar_enabled = True
        # Reduce committed gradients as soon as a batch of weight-gradient tasks has run, without
        # waiting for an all-to-all window: for the device-initiated (fused) transports, whose
        # exchanges never occupy the communication stream.
        self.eager_ar = False
        self.eager_ar_min_bytes = 32 << 20
        # Inside ``no_sync()``: gradients accumulate in the flat buffers, nothing is reduced.
        self.ar_suspended = False
        self.profiling = False
        self.comm_metrics_enabled = False
        # all-reduce configuration
        self.shared_dp_group = None
        self.expert_dp_group = None
        self.shared_dp_world = 1
        self.expert_dp_world = 1
        self.gap_budgets: Dict[str, float] = {}    # region -> ms
        self.shared_ar_bw = 0.0                    # bytes / ms
        self.expert_ar_bw = 0.0
        self.shared_buffer = FlatGradBuffer()
        self.expert_buffer = FlatGradBuffer()
        self.shared_reduce_fn = None
        self.expert_reduce_fn = None
        # dW execution policy specific to this framework
        self.dw_on_side_stream = False
        self.dw_max_ctas = 0
        # queues
        self._dw_queue: Deque[DWTask] = collections.deque()
        self._side_inflight: List[DWTask] = []
        self._pending_param_ar: List[torch.nn.Parameter] = []
        self._a2a_tasks: Dict[int, tuple] = {}
        self._next_task_id = 0
        self._device = None
        self._cuda_ready = False
        self._dw_sync_event = None
        self._ar_done_event = None
        self._current_region: Optional[str] = None
        self._region_start = None
        self._region_records: List[tuple] = []
        self._region_gaps: Dict[str, List[float]] = {}
        self._gap_event_pairs: List[tuple] = []
        self._last_a2a_end = None
        self.reset_comm_metrics()
        # counters
        self.total_dw = self.completed_dw = 0
        self.total_ar = self.completed_ar = 0
        self.ar_during_overlap = 0
        self.ar_submitted_during_bwd = 0
        self.ar_submitted_during_finish = 0
        self._in_finish = False

    def _ensure_device(self, device=None) -> None:
        if self._cuda_ready and (device is None or torch.device(device) == self._device):
            return
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
                else torch.device("cpu")
        sm = get_stream_manager(device)
        if not sm.initialized:
            sm.initialize(device)
        self._device = sm.device
        self._dw_sync_event = make_event(self._device)
        self._ar_done_event = make_event(self._device)
        self._cuda_ready = True

    @property
    def comm_stream(self):
        self._ensure_device()
        return get_stream_manager(self._device).comm_stream

    @property
    def dw_stream(self):
        self._ensure_device()
        return get_stream_manager(self._device).dw_stream

    # ------------------------------------------------------------------ configuration
    def enable(self, device=None) -> None:
        self._ensure_device(device)
        self.enabled = True

    def disable(self) -> None:
        self.enabled = False

    def is_enabled(self) -> bool:
        return self.enabled

    def configure_allreduce(self, enabled: bool = True, shared_dp_group=None, expert_dp_group=None,
                            gap_budgets: Optional[Dict[str, float]] = None,
                            shared_ar_bw: Optional[float] = None,
                            expert_ar_bw: Optional[float] = None,
                            shared_reduce_fn=None, expert_reduce_fn=None) -> None:
        self.ar_enabled = bool(enabled)
        self.shared_dp_group = shared_dp_group
        self.expert_dp_group = expert_dp_group
        init = dist.is_initialized()
        self.shared_dp_world = dist.get_world_size(shared_dp_group) if (init and shared_dp_group is not None) else 1
        self.expert_dp_world = dist.get_world_size(expert_dp_group) if (init and expert_dp_group is not None) else 1
        if gap_budgets is not None:
            self.gap_budgets = dict(gap_budgets)
        if shared_ar_bw is not None:
            self.shared_ar_bw = float(shared_ar_bw)
        if expert_ar_bw is not None:
            self.expert_ar_bw = float(expert_ar_bw)
        self.shared_reduce_fn = shared_reduce_fn or _default_reduce(shared_dp_group)
        self.expert_reduce_fn = expert_reduce_fn or _default_reduce(expert_dp_group)

    def setup_ar_buffer(self, params, accumulate_in_fp32: bool = False, allocator=None) -> None:
        self.shared_buffer.setup(params, accumulate_in_fp32, allocator)

    def setup_expert_ar_buffer(self, params, accumulate_in_fp32: bool = False, allocator=None) -> None:
        self.expert_buffer.setup(params, accumulate_in_fp32, allocator)

    def _buffer_of(self, param) -> Optional[FlatGradBuffer]:
        if param is None:
            return None
        if param in self.shared_buffer:
            return self.shared_buffer
        if param in self.expert_buffer:
            return self.expert_buffer
        return None

    # ------------------------------------------------------------------ dW tasks
    def register_dw_task(self, layer_name: str, layer_id: int, compute_fn: Callable,
                         weight_param=None, needs_ar: bool = True, target_buffer=None,
                         defer: bool = True) -> None:
        """Queue a weight-gradient task; when the scheduler is off it runs right away."""
        task = DWTask(layer_name, layer_id, compute_fn, weight_param, needs_ar, target_buffer, defer)
        self.total_dw += 1
        if not self.enabled:
            self._run_task(task)
            return
        tok = get_overhead_profiler().enter("overhead.bwd_register_dw")
        self._dw_queue.append(task)
        get_overhead_profiler().exit(tok)

    def num_queued_dw_tasks(self) -> int:
        return len(self._dw_queue)

    def _run_task(self, task: DWTask) -> None:
        grad = task.compute_fn()
        param = task.weight_param
        self.completed_dw += 1
        if param is None:
            return
        buf = self._buffer_of(param)
        if buf is not None:
            buf.write_grad(param, grad)
            return
        if grad is None:
            return
        if task.target_buffer is not None:
            task.target_buffer.add_(grad.view_as(task.target_buffer))
        elif param.grad is None:
            param.grad = grad.to(param.dtype).view_as(param).clone() if grad.dtype != param.dtype \
                else grad.view_as(param).clone()
        else:
            param.grad.add_(grad.view_as(param))
        if task.needs_ar and self.enabled:
            self._pending_param_ar.append(param)

    def join_dw_stream(self) -> None:
        """The compute stream waits for every weight-gradient task issued on the side stream; their
        input tensors may be released afterwards."""
        if self._side_inflight:
            current_stream(self._device).wait_stream(self.dw_stream)
            self._side_inflight.clear()

    def _commit(self) -> None:
        cur = current_stream(self._device)
        if self._side_inflight:
            # committed gradients may have been produced on either stream
            self.dw_stream.wait_stream(cur)
            self._dw_sync_event.record(self.dw_stream)
        else:
            self._dw_sync_event.record(cur)
        self.shared_buffer.commit()
        self.expert_buffer.commit()

    def execute_dw_tasks(self, commit_per_task: bool = False,
                         max_defer_tasks: Optional[int] = None) -> int:
        """Run queued tasks in FIFO order.

        At most ``max_defer_tasks`` deferrable tasks run (None = all); tasks registered with
        ``defer=False`` always run.  Deferrable tasks beyond the cap go back to the front of the
        queue in their original order.  Returns the number of tasks executed.
        """
        if not self._dw_queue:
            return 0
        self._ensure_device()
        if not self._in_finish and (not self.stage2_enabled or self.skip_all_dw or
                                    (self.skip_dispatch_dw and self._current_region == "moe_dispatch")):
            # Ablation: nothing runs inside windows except tasks that must not be deferred.
            max_defer_tasks = 0
        tok = get_overhead_profiler().enter("overhead.bwd_execute_dw")
        ran_deferrable = 0
        executed = 0
        kept: List[DWTask] = []
        # Side-stream policy: deferrable tasks run on a low-priority stream behind the work queued so
        # far (their inputs) and the compute stream does NOT wait for them here; it joins at the end
        # of the backward pass (``join_dw_stream``).  Until then the tasks are kept alive, because
        # the tensors their kernels read were allocated on the compute stream and must not be
        # handed out again while those kernels are pending.  The gradient reduction waits for the
        # side stream through ``_dw_sync_event``.
        side = self.dw_on_side_stream and not isinstance(self.dw_stream, NullStream) and not self._in_finish
        if side:
            self.dw_stream.wait_stream(current_stream(self._device))
        while self._dw_queue:
            task = self._dw_queue.popleft()
            if task.defer and max_defer_tasks is not None and ran_deferrable >= max_defer_tasks:
                kept.append(task)
                continue
            if side and task.defer:
                with on_stream(self.dw_stream):
                    self._run_task(task)
                self._side_inflight.append(task)
            else:
                self._run_task(task)
            executed += 1
            if task.defer:
                ran_deferrable += 1
            if commit_per_task:
                self._commit()
                if self.ar_enabled:
                    self._submit_ar_inline(budgeted=False)
        for task in reversed(kept):
            self._dw_queue.appendleft(task)
        if executed and not commit_per_task:
            self._commit()
            if (self.eager_ar and self.ar_enabled and not self._in_finish and
                    (self.shared_buffer.pending_bytes() >= self.eager_ar_min_bytes or
                     (self.expert_dp_world > 1 and self.expert_buffer.pending_bytes() >= self.eager_ar_min_bytes))):
                self._submit_ar_inline(budgeted=False)
        get_overhead_profiler().exit(tok)
        return executed

    # ------------------------------------------------------------------ all-reduce
    def _compute_ar_budget(self) -> tuple:
        """Bytes the shared / expert buffers may reduce in the gap after the current region."""
        if self.fixed_ar_budget > 0:
            total = int(self.fixed_ar_budget)
            exp = min(total, self.expert_buffer.pending_bytes())
            return total - exp, exp
        region = self._current_region or ""
        gap_ms = self.gap_budgets.get(region, 0.0) if self.use_profiled_gaps else 0.0
        if gap_ms <= 0.0:
            return 0, 0
        exp_bytes = 0
        remaining_ms = gap_ms
        if self.expert_dp_world > 1 and self.expert_ar_bw > 0 and self.expert_buffer.has_pending():
            exp_bytes = int(min(self.expert_buffer.pending_bytes(), remaining_ms * self.expert_ar_bw))
            remaining_ms -= exp_bytes / self.expert_ar_bw
        shared_bytes = int(max(0.0, remaining_ms) * self.shared_ar_bw) if self.shared_ar_bw > 0 else 0
        return shared_bytes, exp_bytes

    def _submit_ar_inline(self, budgeted: bool = True) -> int:
        """Reduce committed gradients on the communication stream (behind the dW that made them)."""
        if not self.ar_enabled or self.ar_suspended:
            return 0
        sb, eb = self.shared_buffer, self.expert_buffer
        if not (sb.has_pending() or eb.has_pending() or self._pending_param_ar):
            return 0
        if budgeted:
            shared_budget, expert_budget = self._compute_ar_budget()
            if shared_budget <= 0 and expert_budget <= 0:
                return 0
        else:
            shared_budget = expert_budget = 0  # 0 = unlimited
        tok = get_overhead_profiler().enter("overhead.ar_submit")
        comm = self.comm_stream
        comm.wait_event(self._dw_sync_event)
        scale = 1.0 / self.shared_dp_world
        total = 0
        timing = self.comm_metrics_enabled
        if timing:
            s_evt = make_event(self._device, True)
            s_evt.record(comm)
        with on_stream(comm):
            if eb.has_pending() and self._expert_grads_consumed():
                eb.skip_pending()
            elif eb.has_pending() and (not budgeted or expert_budget > 0):
                # Expert gradients use the same pre-scale as shared ones even when there is a
                # single expert-data-parallel replica (AVG convention of the whole model).
                total += eb.submit_block(self.expert_reduce_fn, expert_budget, scale)
            if sb.has_pending() and (not budgeted or shared_budget > 0):
                total += sb.submit_block(self.shared_reduce_fn, shared_budget, scale)
            if not budgeted and self._pending_param_ar:
                for p in self._pending_param_ar:
                    if p.grad is not None:
                        fn = self.expert_reduce_fn if getattr(p, "allreduce", True) is False else self.shared_reduce_fn
                        fn(p.grad, scale)
                self._pending_param_ar.clear()
        self._ar_done_event.record(comm)
        if timing:
            e_evt = make_event(self._device, True)
            e_evt.record(comm)
            self._ar_event_pairs.append((self._current_region or "dp_tail", s_evt, e_evt))
        if total:
            self.total_ar += 1
            self.completed_ar += 1
            if self._in_finish:
                self.ar_submitted_during_finish += 1
            else:
                self.ar_submitted_during_bwd += 1
                self.ar_during_overlap += 1
        get_overhead_profiler().exit(tok)
        return total

    # ------------------------------------------------------------------ all-to-all
    def _submit(self, fn: Callable, args: tuple) -> int:
        self._ensure_device()
        tok = get_overhead_profiler().enter("overhead.bwd_submit_a2a")
        tid = self._next_task_id
        self._next_task_id += 1
        sm = get_stream_manager(self._device)
        start = sm.get_sync_event(("a2a", 2 * (tid % 4096)), enable_timing=False)
        comm = self.comm_stream
        start.record(current_stream(self._device))
        comm.wait_event(start)
        timing = self.comm_metrics_enabled or self.profiling
        if timing:
            t0 = make_event(self._device, True)
            t0.record(comm)
            if self.profiling and self._last_a2a_end is not None:
                self._gap_event_pairs.append((self._current_region or "", self._last_a2a_end, t0))
        with on_stream(comm):
            result = fn(*args)
        end = make_event(self._device, timing)
        end.record(comm)
        if timing:
            self._a2a_event_pairs.append((self._current_region or "", t0, end))
            self._last_a2a_end = end
        self._a2a_tasks[tid] = (end, result)
        get_overhead_profiler().exit(tok)
        return tid

    def submit_alltoall(self, comm_fn: Callable) -> int:
        return self._submit(comm_fn, ())

    def submit_alltoall_call(self, comm_fn: Callable, *args) -> int:
        return self._submit(comm_fn, args)

    def submit_alltoall_batch(self, comm_fns: list) -> list:
        return [self._submit(fn, ()) for fn in comm_fns]

    def submit_alltoall_batch_call(self, comm_fn: Callable, op_args: list) -> list:
        return [self._submit(comm_fn, tuple(a)) for a in op_args]

    def wait_alltoall(self, task_id: int, num_tasks: int = 1, try_trickle: bool = True):
        """Make the compute stream wait for the given all-to-all(s); returns the last result.

        When no all-to-all remains outstanding the communication stream is idle until the next
        submission: a budgeted slice of the gradient all-reduce is issued into that gap.
        """
        tok = get_overhead_profiler().enter("overhead.bwd_wait_a2a")
        result = None
        cur = current_stream(self._device)
        for tid in range(task_id, task_id + num_tasks):
            ent = self._a2a_tasks.pop(tid, None)
            if ent is None:
                continue
            end, result = ent
            if self.comm_metrics_enabled:
                w0 = make_event(self._device, True)
                w0.record(cur)
            cur.wait_event(end)
            if self.comm_metrics_enabled:
                w1 = make_event(self._device, True)
                w1.record(cur)
                self._visible_wait_pairs.append((self._current_region or "", w0, w1))
        if try_trickle and not self._a2a_tasks and self.enabled and self.ar_enabled and self.pending_ar_enabled:
            self._submit_ar_inline(budgeted=True)
        get_overhead_profiler().exit(tok)
        return result

    def _expert_grads_consumed(self) -> bool:
        """Expert gradients never reach their buffer when the optimizer runs in the weight-gradient
        epilogue of every expert parameter and there are no expert-data-parallel replicas."""
        return getattr(self, "expert_dp_world", 1) <= 1 and self.expert_buffer.consumed_in_backward()

    # ------------------------------------------------------------------ iteration boundaries
    def _reduce_all_sync(self) -> None:
        """F / FB tail: one synchronous reduction of everything that was produced."""
        self._ensure_device()
        scale = 1.0 / self.shared_dp_world
        cur = current_stream(self._device)
        comm = self.comm_stream
        ev = make_event(self._device)
        ev.record(cur)
        comm.wait_event(ev)
        with on_stream(comm):
            if self.expert_buffer.primary is not None:
                if self._expert_grads_consumed():
                    self.expert_buffer.commit_all()
                    self.expert_buffer.skip_pending()
                else:
                    self.expert_buffer.sync_allreduce(self.expert_reduce_fn, scale)
            if self.shared_buffer.primary is not None:
                self.shared_buffer.sync_allreduce(self.shared_reduce_fn, scale)
            for p in self._pending_param_ar:
                if p.grad is not None:
                    fn = self.expert_reduce_fn if getattr(p, "allreduce", True) is False else self.shared_reduce_fn
                    fn(p.grad, scale)
            self._pending_param_ar.clear()
        self._ar_done_event.record(comm)
        cur.wait_event(self._ar_done_event)

    def sync_allreduce_params(self, params) -> None:
        """F mode: reduce ``param.grad`` of every given parameter (scheduler disabled)."""
        self._ensure_device()
        if self.shared_reduce_fn is None:
            self.configure_allreduce(self.ar_enabled, self.shared_dp_group, self.expert_dp_group)
        scale = 1.0 / self.shared_dp_world
        for p in params:
            g = getattr(p, "grad", None)
            if g is None:
                continue
            fn = self.expert_reduce_fn if getattr(p, "allreduce", True) is False else self.shared_reduce_fn
            fn(g, scale)

    def finish_batch(self) -> None:
        """Drain the queue at the end of the backward pass and finish the gradient reduction."""
        if not self.enabled:
            return
        self._ensure_device()
        self._in_finish = True
        prev_region, self._current_region = self._current_region, "dp_tail"
        self.join_dw_stream()
        try:
            if self.ar_enabled:
                self.execute_dw_tasks(commit_per_task=True)
                self._commit()
                self.shared_buffer.commit_all()
                self.expert_buffer.commit_all()
                self._submit_ar_inline(budgeted=False)
                cur = current_stream(self._device)
                if self.comm_metrics_enabled:
                    w0 = make_event(self._device, True)
                    w0.record(cur)
                cur.wait_event(self._ar_done_event)
                if self.comm_metrics_enabled:
                    w1 = make_event(self._device, True)
                    w1.record(cur)
                    self._ar_visible_wait_pairs.append(("dp_tail", w0, w1))
            else:
                self.execute_dw_tasks()
                self._commit()
                if self.shared_dp_world > 1 or self.expert_dp_world > 1 or self._pending_param_ar:
                    if self.shared_reduce_fn is None:
                        self.configure_allreduce(False, self.shared_dp_group, self.expert_dp_group)
                    self._reduce_all_sync()
        finally:
            self._in_finish = False
            self._current_region = prev_region

    @contextlib.contextmanager
    def no_sync(self):
        """Gradient accumulation: run every micro-batch but the last inside this context.

        A slice of the flat buffer is reduced once, as soon as its gradients are committed; a
        micro-batch that adds to it afterwards would be left out of the reduction.  Inside the
        context nothing is reduced.  On exit the weight-gradient queue is drained (so that no task
        of an earlier micro-batch can mark a parameter as produced during the last one) and the
        cursors start over: the last micro-batch then commits and reduces every parameter after its
        final accumulation.  The reference reduces during every backward pass and has no
        accumulation mode (fluid/core/scheduler.py:188-213)."""
        prev = self.ar_suspended
        self.ar_suspended = True
        try:
            yield self
        finally:
            if self.enabled and not prev:
                if self._dw_queue:
                    self.execute_dw_tasks()          # still suspended: this commit reduces nothing
                self.shared_buffer.reset_cursors()
                self.expert_buffer.reset_cursors()
            self.ar_suspended = prev

    def clear_iteration(self) -> None:
        """Wait for anything outstanding and reset per-iteration state."""
        if self._cuda_ready:
            cur = current_stream(self._device)
            for end, _ in self._a2a_tasks.values():
                cur.wait_event(end)
            if self._ar_done_event is not None:
                cur.wait_event(self._ar_done_event)
        self._a2a_tasks.clear()
        self._next_task_id = 0
        if self._cuda_ready:
            self.join_dw_stream()
        self._dw_queue.clear()
        self._pending_param_ar.clear()
        self.shared_buffer.reset_cursors()
        self.expert_buffer.reset_cursors()
        self._current_region = None
        self._last_a2a_end = None

    # ------------------------------------------------------------------ regions / profiling
    def begin_region(self, name: str) -> None:
        self._current_region = name
        if self.profiling:
            self._ensure_device()
            ev = make_event(self._device, True)
            ev.record(current_stream(self._device))
            self._region_start = (name, ev, len(self._a2a_event_pairs))
            self._last_a2a_end = None

    def end_region(self) -> None:
        if not self.cross_region_flow and self.enabled and self._dw_queue and not self._in_finish:
            # Ablation: no weight-gradient task outlives the region that queued or inherited it;
            # the queue is drained at every region boundary (fluid/core/scheduler.py:1048-1052).
            self.execute_dw_tasks(commit_per_task=False)
        if self.profiling and self._region_start is not None:
            name, s_ev, first_pair = self._region_start
            e_ev = make_event(self._device, True)
            e_ev.record(current_stream(self._device))
            self._region_records.append((name, s_ev, e_ev, first_pair, len(self._a2a_event_pairs)))
            self._region_start = None
        self._current_region = None

    def get_region_profiles(self) -> Dict[str, Dict[str, float]]:
        """Per-region ``T_region`` (compute-stream span), ``T_comm`` (sum of its all-to-alls) and
        ``T_comp`` = T_region - exposed wait; averaged over the recorded iterations."""
        if self._cuda_ready and self._device.type == "cuda":
            torch.cuda.synchronize(self._device)
        acc: Dict[str, Dict[str, float]] = {}
        for name, s_ev, e_ev, lo, hi in self._region_records:
            d = acc.setdefault(name, {"T_region": 0.0, "T_comm": 0.0, "n": 0})
            d["T_region"] += s_ev.elapsed_time(e_ev)
            d["T_comm"] += sum(s.elapsed_time(e) for _, s, e in self._a2a_event_pairs[lo:hi])
            d["n"] += 1
        out = {}
        for name, d in acc.items():
            n = max(1, d["n"])
            out[name] = {"T_region": d["T_region"] / n, "T_comm": d["T_comm"] / n,
                         "T_comp": max(0.0, (d["T_region"] - d["T_comm"]) / n), "n": d["n"]}
        return out

    def reset_gap_times(self) -> None:
        self._gap_event_pairs = []
        self._region_gaps = {}
        self._last_a2a_end = None
        self._region_records = []

    def process_gap_events(self) -> Dict[str, List[float]]:
        if self._cuda_ready and self._device.type == "cuda":
            torch.cuda.synchronize(self._device)
        for region, end_prev, start_next in self._gap_event_pairs:
            self._region_gaps.setdefault(region, []).append(end_prev.elapsed_time(start_next))
        self._gap_event_pairs = []
        return self._region_gaps

    # ------------------------------------------------------------------ exposed-communication metrics
    def set_comm_metrics_enabled(self, enabled: bool) -> None:
        self.comm_metrics_enabled = bool(enabled)

    def reset_comm_metrics(self) -> None:
        self._a2a_event_pairs: List[tuple] = []
        self._visible_wait_pairs: List[tuple] = []
        self._ar_event_pairs: List[tuple] = []
        self._ar_visible_wait_pairs: List[tuple] = []
        self._qr_samples: List[float] = []

    def begin_fwd_comm(self, comm_stream):
        if not self.comm_metrics_enabled:
            return None
        self._ensure_device()
        ev = make_event(self._device, True)
        ev.record(comm_stream)
        return ev

    def end_fwd_comm(self, region: str, start_evt, comm_stream, end_evt=None) -> None:
        if not self.comm_metrics_enabled or start_evt is None:
            return
        if end_evt is None:
            end_evt = make_event(self._device, True)
            end_evt.record(comm_stream)
        self._a2a_event_pairs.append((region, start_evt, end_evt))

    def record_fwd_wait(self, region: str, end_evt) -> None:
        """Make the compute stream wait for ``end_evt`` (always: the forward pairwise exchanges
        rely on it, whether or not the scheduler was ever enabled) and, with metrics on, bracket
        the wait so that its exposed part can be measured."""
        if end_evt is None:
            return
        if not self._cuda_ready:
            self._ensure_device()
        cur = current_stream(self._device)
        if not self.comm_metrics_enabled:
            cur.wait_event(end_evt)
            return
        w0 = make_event(self._device, True)
        w0.record(cur)
        cur.wait_event(end_evt)
        w1 = make_event(self._device, True)
        w1.record(cur)
        self._visible_wait_pairs.append((region, w0, w1))

    def record_Qr_sample(self, compute_ms: float) -> None:
        if self.comm_metrics_enabled:
            self._qr_samples.append(float(compute_ms))

    def get_avg_Qr_ms(self) -> float:
        return sum(self._qr_samples) / len(self._qr_samples) if self._qr_samples else 0.0

    def get_comm_metrics(self) -> dict:
        """Total and exposed all-to-all / all-reduce time per region (exposed = min(wait, total))."""
        if self._cuda_ready and self._device.type == "cuda":
            torch.cuda.synchronize(self._device)
        per: Dict[str, Dict[str, float]] = {}

        def bucket(r):
            return per.setdefault(r, dict(a2a_total_ms=0.0, a2a_wait_ms=0.0, a2a_visible_ms=0.0,
                                          ar_total_ms=0.0, ar_wait_ms=0.0, ar_visible_ms=0.0))
        for r, s, e in self._a2a_event_pairs:
            bucket(r)["a2a_total_ms"] += s.elapsed_time(e)
        for r, s, e in self._visible_wait_pairs:
            bucket(r)["a2a_wait_ms"] += s.elapsed_time(e)
        for r, s, e in self._ar_event_pairs:
            bucket(r)["ar_total_ms"] += s.elapsed_time(e)
        for r, s, e in self._ar_visible_wait_pairs:
            bucket(r)["ar_wait_ms"] += s.elapsed_time(e)
        for b in per.values():
            b["a2a_visible_ms"] = min(b["a2a_wait_ms"], b["a2a_total_ms"])
            b["ar_visible_ms"] = min(b["ar_wait_ms"], b["ar_total_ms"])
        a2a_t = sum(b["a2a_total_ms"] for b in per.values())
        a2a_v = sum(b["a2a_visible_ms"] for b in per.values())
        ar_t = sum(b["ar_total_ms"] for b in per.values())
        ar_v = sum(b["ar_visible_ms"] for b in per.values())
        return {
            "a2a_total_ms": a2a_t, "a2a_visible_ms": a2a_v,
            "a2a_overlap_ratio": 0.0 if a2a_t <= 1e-9 else max(0.0, min(1.0, 1.0 - a2a_v / a2a_t)),
            "n_a2a": len(self._a2a_event_pairs), "n_waits": len(self._visible_wait_pairs),
            "ar_total_ms": ar_t, "ar_visible_ms": ar_v,
            "ar_overlap_ratio": 0.0 if ar_t <= 1e-9 else max(0.0, min(1.0, 1.0 - ar_v / ar_t)),
            "n_ar": len(self._ar_event_pairs), "per_region": per,
        }

    @staticmethod
    def measure_ar_bandwidth(ar_group=None, sizes_mb=(1, 2, 4, 8, 16, 32, 64, 96, 128), warmup=5,
                             repeat=20, dtype=torch.float32, reduce_fn=None) -> dict:
        """All-reduce latency / bandwidth sweep used to convert gap budgets (ms) into bytes."""
        cuda = torch.cuda.is_available()
        device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
        reduce_fn = reduce_fn or (lambda t: dist.all_reduce(t, group=ar_group)
                                  if dist.is_initialized() else None)
        res = {"sizes_mb": [], "bw_GBps": [], "latency_ms": []}
        esize = torch.empty((), dtype=dtype).element_size()
        for mb in sizes_mb:
            n = int(mb * 1024 * 1024 / esize)
            t = torch.zeros(n, dtype=dtype, device=device)
            for _ in range(warmup):
                reduce_fn(t)
            s, e = make_event(device, True), make_event(device, True)
            if cuda:
                torch.cuda.synchronize()
            s.record()
            for _ in range(repeat):
                reduce_fn(t)
            e.record()
            if cuda:
                torch.cuda.synchronize()
            lat = s.elapsed_time(e) / repeat
            res["sizes_mb"].append(mb)
            res["latency_ms"].append(lat)
            res["bw_GBps"].append((n * esize / 1e9) / (lat / 1e3) if lat > 0 else 0.0)
        res["peak_bw_GBps"] = max(res["bw_GBps"]) if res["bw_GBps"] else 0.0
        return res

    def get_stats(self) -> dict:
        return {
            "total_dw_tasks": self.total_dw, "completed_dw_tasks": self.completed_dw,
            "total_ar_tasks": self.total_ar, "completed_ar_tasks": self.completed_ar,
            "ar_during_gap": self.ar_during_overlap,
            "ar_submitted_during_bwd": self.ar_submitted_during_bwd,
            "ar_submitted_during_finish": self.ar_submitted_during_finish,
            "pending_dw_at_finish": len(self._dw_queue),
            "region_gaps": dict(self._region_gaps),
            "shared_ar_bw": self.shared_ar_bw, "expert_ar_bw": self.expert_ar_bw,
        }

    @classmethod
    def reset(cls) -> None:
        cls._instance = None


def get_backward_scheduler() -> BackwardScheduler:
    return BackwardScheduler()
