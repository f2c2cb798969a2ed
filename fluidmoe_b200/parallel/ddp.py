"""Data-parallel wrapper and optimizer wrapper around the backward scheduler.

``FluidDDP`` routes gradients three ways, as the reference's wrapper does (fluid/setup.py:24-381):
block parameters into the scheduler's flat buffers (dense and expert separately, fp32
accumulation), the head / final-norm parameters to the front of the dense buffer so that the
earliest communication gaps can reduce them, and everything else (embeddings) into a private
contiguous fp32 buffer that is reduced after ``finish_batch``.  Megatron is not required; when it
is installed ``setup_model_and_optimizer`` mirrors Megatron's function of the same name.
"""
from __future__ import annotations

import os
from typing import Callable, Iterable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .scheduler import BackwardScheduler, get_backward_scheduler

_GAP_ENV = {"moe_combine": "FLUIDMOE_GAP_MOE_COMBINE", "moe_dispatch": "FLUIDMOE_GAP_MOE_DISPATCH",
            "attn_proj": "FLUIDMOE_GAP_ATTN_PROJ", "attn_qkv": "FLUIDMOE_GAP_ATTN_QKV"}


def _env_float(name: str, default: float) -> float:
    try:
        return float(os.environ.get(name, default))
    except ValueError:
        return default


class FluidDDP(nn.Module):
    def __init__(self, config, module: nn.Module, scheduler: Optional[BackwardScheduler] = None,
                 dp_cp_group=None, expert_dp_group=None, accumulate_in_fp32: bool = True,
                 ar_enabled: bool = True, gap_budgets: Optional[dict] = None,
                 shared_ar_bw: Optional[float] = None, expert_ar_bw: Optional[float] = None,
                 shared_reduce_fn=None, expert_reduce_fn=None, allocator=None, eager_ar: Optional[bool] = None,
                 grad_reduce: Optional[str] = None):
        super().__init__()
        self.config = config
        self.module = module
        self.scheduler = scheduler or get_backward_scheduler()
        self.dp_cp_group, self.expert_dp_group = dp_cp_group, expert_dp_group
        self.dp_world = dist.get_world_size(dp_cp_group) if (dist.is_initialized() and dp_cp_group is not None) else 1
        self.fused_ctx = None
        for mod in module.modules():
            if getattr(mod, "fused_ctx", None) is not None:
                self.fused_ctx = mod.fused_ctx
                break
        # Dense-gradient reduction: "nccl" (library all-reduce) or "symm" (this library's two-shot
        # kernel over peer memory on a flat buffer that lives in the symmetric heap); the latter
        # needs the device-initiated transport and a dense data-parallel group equal to its group.
        mode = (grad_reduce or os.environ.get("FLUIDMOE_GRAD_REDUCE", "nccl")).lower()
        self.grad_reducer = None
        if mode == "symm" and shared_reduce_fn is None and allocator is None and self.fused_ctx is not None \
                and self.dp_world == self.fused_ctx.world and self.dp_world > 1:
            from .scheduler import _default_reduce
            from .symm import SymmGradReducer
            self.grad_reducer = SymmGradReducer(self.fused_ctx.heap, fallback=_default_reduce(dp_cp_group))
            shared_reduce_fn = self.grad_reducer.reduce
            shared_allocator = self.grad_reducer.allocator
        else:
            shared_allocator = allocator
        self.grad_reduce_mode = "symm" if self.grad_reducer is not None else "nccl"
        self._configure_scheduler(accumulate_in_fp32, ar_enabled, gap_budgets, shared_ar_bw, expert_ar_bw,
                                  shared_reduce_fn, expert_reduce_fn, allocator, shared_allocator)
        if self.grad_reducer is not None:
            self.fused_ctx.heap.sync_group()
        self._setup_other_params()
        # With the device-initiated transports there are no all-to-all windows to trickle the gradient
        # reduction into: start it as soon as gradients are committed instead.
        self.scheduler.eager_ar = (self.fused_ctx is not None) if eager_ar is None else bool(eager_ar)

    # ------------------------------------------------------------------ configuration
    def _decoder_layers(self):
        m = self.module
        for path in ("decoder.layers", "layers", "module.decoder.layers"):
            obj = m
            try:
                for part in path.split("."):
                    obj = getattr(obj, part)
                return list(obj)
            except AttributeError:
                continue
        return []

    def _configure_scheduler(self, fp32, ar_enabled, gap_budgets, shared_bw, expert_bw, s_fn, e_fn, allocator,
                             shared_allocator=None):
        sched = self.scheduler
        gaps = dict(gap_budgets or {})
        for region, env in _GAP_ENV.items():
            if env in os.environ:
                gaps[region] = _env_float(env, gaps.get(region, 0.0))
        shared_bw = _env_float("FLUIDMOE_SHARED_AR_BW", shared_bw if shared_bw is not None else 0.0)
        expert_bw = _env_float("FLUIDMOE_EXPERT_AR_BW", expert_bw if expert_bw is not None else 0.0)
        sched.configure_allreduce(ar_enabled, self.dp_cp_group, self.expert_dp_group, gaps, shared_bw,
                                  expert_bw, s_fn, e_fn)
        shared: List[nn.Parameter] = []
        expert: List[nn.Parameter] = []
        inline = os.environ.get("FLUIDMOE_DISABLE_MODEL_LEVEL_INLINE_AR", "0") != "1"
        if inline:
            for name in ("lm_head", "output_layer", "final_norm_weight", "final_norm_bias", "final_layernorm"):
                obj = getattr(self.module, name, None)
                if isinstance(obj, nn.Parameter):
                    shared.append(obj)
                elif isinstance(obj, nn.Module):
                    shared += list(obj.parameters())
        for layer in reversed(self._decoder_layers()):
            inner = getattr(layer, "layer", layer)
            ex = [p for p in (getattr(inner, "moe_w2", None), getattr(inner, "moe_w1", None)) if p is not None]
            expert += ex
            order = ("router_weight", "shared_w2", "shared_w1", "ln2_weight", "ln2_bias", "proj_weight",
                     "qkv_weight", "ln1_weight", "ln1_bias")
            shared += [getattr(inner, n) for n in order if getattr(inner, n, None) is not None]
        self._scheduler_params = {id(p) for p in shared + expert}
        sched.setup_ar_buffer(shared, fp32, shared_allocator if shared_allocator is not None else allocator)
        sched.setup_expert_ar_buffer(expert, fp32, allocator)

    def _setup_other_params(self) -> None:
        """Parameters outside the scheduler get a contiguous fp32 gradient buffer filled by
        post-accumulate hooks and reduced once per iteration."""
        others = [p for p in self.module.parameters() if p.requires_grad and id(p) not in self._scheduler_params]
        self._others = others
        n = sum(p.numel() for p in others)
        self._grad_buffer = torch.zeros(n, dtype=torch.float32, device=others[0].device) if others else None
        off = 0
        for p in others:
            p.main_grad = self._grad_buffer[off:off + p.numel()].view(p.shape)
            off += p.numel()

            def hook(param):
                if param.grad is not None:
                    param.main_grad.add_(param.grad.float())
                    param.grad = None
            p.register_post_accumulate_grad_hook(hook)

    # ------------------------------------------------------------------ training-loop API
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def zero_grad_buffer(self) -> None:
        for p in self.module.parameters():
            p.grad = None
            if hasattr(p, "_ar_buf_written"):
                p._ar_buf_written = False
        self.scheduler.shared_buffer.reset_cursors()
        self.scheduler.expert_buffer.reset_cursors()
        if self._grad_buffer is not None:
            self._grad_buffer.zero_()

    def no_sync(self):
        """Context for every micro-batch but the last of an accumulated step: gradients add up in
        the flat buffers and nothing is reduced (see ``BackwardScheduler.no_sync``).  Call
        ``finish_grad_sync`` once, after the last micro-batch."""
        return self.scheduler.no_sync()

    def finish_grad_sync(self, force_all_reduce: bool = False) -> None:
        """Run what is left of the weight-gradient queue and finish every gradient reduction.
        ``force_all_reduce`` is accepted for callers written against Megatron's DDP interface
        (fluid/setup.py:332); the reduction here is always a full all-reduce."""
        self.scheduler.finish_batch()
        fused = getattr(self, "fused_ctx", None)
        if fused is not None:
            fused.iteration_barrier()   # peers may not reuse this iteration's buffers before here
        if not self.scheduler.is_enabled():
            ps = [p for p in self.module.parameters() if id(p) in self._scheduler_params]
            self.scheduler.sync_allreduce_params(ps)
        if self._grad_buffer is not None and self.dp_world > 1:
            self._grad_buffer.mul_(1.0 / self.dp_world)
            dist.all_reduce(self._grad_buffer, group=self.dp_cp_group)

    def scale_gradients(self, scale: float) -> None:
        self.scheduler.shared_buffer.scale_pending(scale)
        self.scheduler.expert_buffer.scale_pending(scale)
        if self._grad_buffer is not None:
            self._grad_buffer.mul_(scale)

    def broadcast_params(self) -> None:
        if not dist.is_initialized() or self.dp_world == 1:
            return
        src = dist.get_global_rank(self.dp_cp_group, 0) if self.dp_cp_group is not None else 0
        for p in self.module.parameters():
            if getattr(p, "allreduce", True):
                dist.broadcast(p.data, src=src, group=self.dp_cp_group)

    def state_dict(self, *args, **kwargs):
        return self.module.state_dict(*args, **kwargs)

    def load_state_dict(self, state_dict, *args, **kwargs):
        return self.module.load_state_dict(state_dict, *args, **kwargs)

    def sharded_state_dict(self, *args, **kwargs):
        fn = getattr(self.module, "sharded_state_dict", None)
        return fn(*args, **kwargs) if fn is not None else self.module.state_dict()


class FluidOptimizerWrapper:
    """``step()`` runs the wrapped optimizer and then resets the scheduler for the next iteration
    (fluid/setup.py:388-418)."""

    def __init__(self, optimizer, scheduler: Optional[BackwardScheduler] = None):
        self._optimizer = optimizer
        self._scheduler = scheduler or get_backward_scheduler()

    @property
    def optimizer(self):
        return self._optimizer

    @property
    def scheduler(self) -> BackwardScheduler:
        return self._scheduler

    def step(self, *args, **kwargs):
        out = self._optimizer.step(*args, **kwargs)
        self._scheduler.clear_iteration()
        return out

    def zero_grad(self, *args, **kwargs):
        return self._optimizer.zero_grad(*args, **kwargs)

    # Everything else is the wrapped optimizer's: reads fall through, and so do writes of public
    # attributes (a training loop that sets ``opt.param_groups`` or a flag reaches the optimizer
    # itself, fluid/setup.py:403-410); only names with a leading underscore live on the wrapper.
    def __getattr__(self, name):
        if name in ("_optimizer", "_scheduler"):     # not set yet (unpickling, failed __init__)
            raise AttributeError(name)
        return getattr(self._optimizer, name)

    def __setattr__(self, name, value):
        if name.startswith("_"):
            object.__setattr__(self, name, value)
        else:
            setattr(self._optimizer, name, value)


def setup_model_and_optimizer(model_provider_func: Callable, model_type=None, checkpointing_context=None,
                              optimizer_factory: Optional[Callable] = None, parallel_ctx=None, **ddp_kwargs):
    """Build ``(model list, optimizer, lr scheduler)``.

    With megatron-core installed and initialised this mirrors Megatron's function (Float16 wrap,
    FluidDDP, Megatron optimizer, checkpoint load).  Without it, ``model_provider_func()`` returns
    the model, which is wrapped in FluidDDP and paired with this library's fused Adam (or with
    ``optimizer_factory(params)``)."""
    sched = get_backward_scheduler()
    sched.enable()
    try:
        from megatron.training import get_args  # type: ignore
        from megatron.core.optimizer import OptimizerConfig, get_megatron_optimizer  # type: ignore
        args = get_args()
        have_megatron = True
    except Exception:  # noqa: BLE001 - megatron absent or not initialised
        have_megatron = False
    if have_megatron:
        from megatron.core import mpu  # type: ignore
        model = model_provider_func(pre_process=True, post_process=True)
        if getattr(args, "bf16", False):
            model = model.bfloat16()
        model = model.cuda()
        ddp = FluidDDP(None, model, sched, dp_cp_group=mpu.get_data_parallel_group(with_context_parallel=True),
                       expert_dp_group=mpu.get_expert_data_parallel_group(), **ddp_kwargs)
        cfg = OptimizerConfig(optimizer="adam", lr=args.lr, weight_decay=args.weight_decay, bf16=args.bf16,
                              use_distributed_optimizer=False)
        opt = FluidOptimizerWrapper(get_megatron_optimizer(cfg, [ddp]), sched)
        return [ddp], opt, None
    model = model_provider_func()
    pc = parallel_ctx
    ddp = FluidDDP(None, model, sched, dp_cp_group=getattr(pc, "dp_cp_group", None),
                   expert_dp_group=getattr(pc, "expert_dp_group", None), **ddp_kwargs)
    if optimizer_factory is None:
        from ..ops.optim import FusedAdam
        optimizer_factory = lambda ps: FusedAdam(ps, lr=1e-4)  # noqa: E731
    opt = FluidOptimizerWrapper(optimizer_factory(list(model.parameters())), sched)
    return [ddp], opt, None
