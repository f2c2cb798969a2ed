"""LayerNorm / RMSNorm forward and backward (statistics in fp32, saved for the backward).

The reference uses Transformer Engine's LayerNorm with a PyTorch fallback
(fluid/core/te_ops.py:43-140); RMSNorm has no counterpart there.  The backward can fold the
residual-branch gradient into ``dx`` (fluid/layer/transformer.py:672,764 do that as a separate add).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native


def norm_fwd(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float = 1e-5,
             kind: str = "layernorm") -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor]:
    """x: [T, H].  Returns ``(y, mean or None, rstd)``; kind is ``layernorm`` or ``rmsnorm``."""
    if _native.use_native(x) and hasattr(_native.lib(), "norm_fwd"):
        from . import elementwise
        res = elementwise.norm_fwd(x, weight, bias, eps, kind)
        if res is not None:
            return res
    xf = x.float()
    if kind == "layernorm":
        mean = xf.mean(-1)
        var = xf.var(-1, unbiased=False)
        rstd = torch.rsqrt(var + eps)
        y = (xf - mean.unsqueeze(-1)) * rstd.unsqueeze(-1) * weight.float()
        if bias is not None:
            y = y + bias.float()
        return y.to(x.dtype), mean, rstd
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    y = xf * rstd.unsqueeze(-1) * weight.float()
    return y.to(x.dtype), None, rstd


def norm_bwd(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, mean: Optional[torch.Tensor],
             rstd: torch.Tensor, kind: str = "layernorm", has_bias: bool = True,
             residual_grad: Optional[torch.Tensor] = None):
    """Returns ``(dx (+ residual_grad), dweight fp32, dbias fp32 or None)``."""
    if _native.use_native(dy, x) and hasattr(_native.lib(), "norm_bwd"):
        from . import elementwise
        res = elementwise.norm_bwd(dy, x, weight, mean, rstd, kind, has_bias, residual_grad)
        if res is not None:
            return res
    dyf, xf, w = dy.float(), x.float(), weight.float()
    r = rstd.unsqueeze(-1)
    if kind == "layernorm":
        xhat = (xf - mean.unsqueeze(-1)) * r
        g = dyf * w
        c1 = (g * xhat).mean(-1, keepdim=True)
        c2 = g.mean(-1, keepdim=True)
        dx = (g - c2 - xhat * c1) * r
        dw = (dyf * xhat).sum(0)
        db = dyf.sum(0) if has_bias else None
    else:
        xhat = xf * r
        g = dyf * w
        c1 = (g * xhat).mean(-1, keepdim=True)
        dx = (g - xhat * c1) * r
        dw = (dyf * xhat).sum(0)
        db = None
    if residual_grad is not None:
        dx = dx + residual_grad.float()
    return dx.to(x.dtype), dw, db
