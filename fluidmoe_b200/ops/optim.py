"""Fused Adam(W) over flat gradient buffers.

The scheduler accumulates gradients in flat fp32 buffers (``param.main_grad``), so the optimizer
walks those buffers directly: one kernel per parameter, bf16 parameter updated in place, fp32
moments (and an optional fp32 master copy).  CPU tensors take a PyTorch path with the same math.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch

from .. import _native


class FusedAdam:
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0, master_weights: bool = False,
                 state_dtype: torch.dtype = torch.float32):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.step_count = 0
        self.state = {}
        self.master_weights = master_weights
        self.state_dtype = state_dtype   # fp32, or bf16 moments as torch.optim.AdamW keeps for bf16 parameters
        self.param_groups = [dict(params=self.params, lr=lr)]
        self.fused_wgrad_params = 0

    # ------------------------------------------------------------------ optimizer in the backward pass
    def fuse_into_backward(self, params: Optional[Iterable[torch.nn.Parameter]] = None,
                           mode: str = "epilogue") -> int:
        """Run this optimizer inside the backward pass for the given parameters (default: every
        expert weight, i.e. parameters marked ``allreduce = False``); ``step`` then skips them.

        ``mode="epilogue"``: the weight-gradient GEMM applies the update in its epilogue
        (``ops.gemm.grouped_gemm_wgrad_adam``), the gradient is never stored.
        ``mode="stream"``: the weight-gradient GEMM stores the gradient as usual and a small-CTA Adam
        kernel is queued behind it on a side stream, where it runs under the tensor-bound kernels of
        the following layers (``ops.elementwise.adam_background``).

        The caller promises one micro-batch per optimizer step, no gradient clipping and no
        data-parallel replicas of these parameters.  Needs bf16 parameters and bf16 moments without
        master weights; returns the number of parameters taken."""
        assert mode in ("epilogue", "stream")
        if self.master_weights or self.state_dtype != torch.bfloat16:
            return 0
        chosen = list(params) if params is not None else [p for p in self.params
                                                          if getattr(p, "allreduce", True) is False]
        n = 0
        for p in chosen:
            if p.dtype == torch.bfloat16 and p.dim() == 3 and p.is_contiguous():
                p._fused_adam = self
                p._fused_update_done = False
                n += 1
        self.fused_wgrad_params = n
        self.fused_mode = mode
        return n

    def update_on_stream(self, p) -> None:
        """``p.main_grad`` holds the complete gradient (written by kernels already queued on the
        current stream): queue the Adam kernel for ``p`` behind them on the optimizer stream."""
        st = self._state(p)
        b1, b2 = self.betas
        g = p.main_grad
        if not (p.is_cuda and _native.available() and g.dtype == torch.float32):
            self._update_reference(p, g.float(), st, self.step_count + 1, 1.0)
            p._fused_update_done = True
            return
        from . import elementwise
        if getattr(self, "_opt_stream", None) is None:
            self._opt_stream = torch.cuda.Stream(device=p.device)
            self._pending_events = []
        ready = torch.cuda.Event()
        ready.record()
        self._opt_stream.wait_event(ready)
        elementwise.adam_background(p.data.view(-1), g.view(-1), st["m"].view(-1), st["v"].view(-1), self.lr, b1, b2,
                                    self.eps, self.weight_decay, self.step_count + 1,
                                    stream=self._opt_stream.cuda_stream)
        done = torch.cuda.Event()
        done.record(self._opt_stream)
        self._pending_events.append(done)
        p._fused_update_done = True

    def _update_reference(self, p, gf, st, step, grad_scale) -> None:
        b1, b2 = self.betas
        gf = gf * grad_scale
        w = st["master"] if st["master"] is not None else p.data.float()
        m32 = st["m"].float().mul_(b1).add_(gf, alpha=1 - b1)
        v32 = st["v"].float().mul_(b2).addcmul_(gf, gf, value=1 - b2)
        st["m"].copy_(m32)
        st["v"].copy_(v32)
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        upd = (m32 / bc1) / ((v32 / bc2).sqrt() + self.eps) + self.weight_decay * w
        w = w - self.lr * upd
        if st["master"] is not None:
            st["master"].copy_(w)
        p.data.copy_(w.to(p.dtype))

    def wgrad_update(self, p, a, dy, num_groups, grad_scale: float = 1.0, **rows_kw) -> None:
        """Called by a weight-gradient task instead of storing the gradient of ``p``."""
        from . import gemm
        st = self._state(p)
        b1, b2 = self.betas
        with torch.no_grad():
            gemm.grouped_gemm_wgrad_adam(a, dy, num_groups, p.data, st["m"], st["v"], lr=self.lr, beta1=b1,
                                         beta2=b2, eps=self.eps, weight_decay=self.weight_decay,
                                         step=self.step_count + 1, grad_scale=grad_scale, **rows_kw)
        p._fused_update_done = True

    def _state(self, p):
        st = self.state.get(id(p))
        if st is None:
            st = dict(m=torch.zeros(p.shape, dtype=self.state_dtype, device=p.device),
                      v=torch.zeros(p.shape, dtype=self.state_dtype, device=p.device),
                      master=p.detach().float().clone() if self.master_weights else None)
            self.state[id(p)] = st
        return st

    @staticmethod
    def _grad_of(p) -> Optional[torch.Tensor]:
        g = getattr(p, "main_grad", None)
        if g is not None and getattr(p, "_ar_buf_written", True):
            return g
        return p.grad

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        for ev in getattr(self, "_pending_events", []):     # updates queued on the optimizer stream
            torch.cuda.current_stream().wait_event(ev)
        if getattr(self, "_pending_events", None):
            self._pending_events.clear()
        self.step_count += 1
        b1, b2 = self.betas
        for p in self.params:
            if getattr(p, "_fused_update_done", False):
                p._fused_update_done = False      # updated by its weight-gradient GEMM already
                continue
            g = self._grad_of(p)
            if g is None:
                continue
            st = self._state(p)
            if p.is_cuda and p.dtype == torch.bfloat16 and g.dtype == torch.float32 and _native.available() \
                    and p.is_contiguous() and g.is_contiguous():
                from . import elementwise
                elementwise.adam_step(p.data, st["master"], g, st["m"], st["v"], self.lr, b1, b2, self.eps,
                                      self.weight_decay, self.step_count, grad_scale)
                continue
            gf = g.float() * grad_scale
            w = st["master"] if st["master"] is not None else p.data.float()
            m32 = st["m"].float().mul_(b1).add_(gf, alpha=1 - b1)
            v32 = st["v"].float().mul_(b2).addcmul_(gf, gf, value=1 - b2)
            st["m"].copy_(m32)
            st["v"].copy_(v32)
            bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
            upd = (m32 / bc1) / ((v32 / bc2).sqrt() + self.eps) + self.weight_decay * w
            w = w - self.lr * upd
            if st["master"] is not None:
                st["master"].copy_(w)
            p.data.copy_(w.to(p.dtype))

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            p.grad = None
            if hasattr(p, "_ar_buf_written"):
                p._ar_buf_written = False

    def state_dict(self):
        """Step count and per-parameter moments, keyed by the parameter's position; tensors are
        detached host copies so that the result can be written with ``torch.save`` as is."""
        return dict(step=self.step_count,
                    state={i: {k: (v.detach().cpu() if torch.is_tensor(v) else v)
                               for k, v in self.state.get(id(p), {}).items()}
                           for i, p in enumerate(self.params)})

    def load_state_dict(self, sd) -> None:
        """Install saved moments (and master copies).  Every tensor is moved to its parameter's
        device and to this optimizer's state dtype first: a checkpoint is read with
        ``map_location='cpu'``, and the kernels take raw pointers, so a host tensor left in the state
        of a CUDA parameter would be dereferenced on the device."""
        self.step_count = int(sd["step"])
        for i, p in enumerate(self.params):
            saved = sd["state"].get(i) or sd["state"].get(str(i))
            if not saved:
                continue
            st = {}
            for key in ("m", "v"):
                t = saved[key]
                if tuple(t.shape) != tuple(p.shape):
                    raise ValueError(f"optimizer state '{key}' of parameter {i} has shape {tuple(t.shape)}, "
                                     f"the parameter has {tuple(p.shape)}")
                st[key] = t.to(device=p.device, dtype=self.state_dtype).contiguous()
            master = saved.get("master")
            if self.master_weights:
                if master is not None and tuple(master.shape) != tuple(p.shape):
                    raise ValueError(f"master copy of parameter {i} has shape {tuple(master.shape)}, "
                                     f"the parameter has {tuple(p.shape)}")
                st["master"] = (master.to(device=p.device, dtype=torch.float32).contiguous()
                                if master is not None else p.detach().float().clone())
            else:
                st["master"] = None
            self.state[id(p)] = st
