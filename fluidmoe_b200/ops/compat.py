"""Functional wrappers under the names the reference gives its Transformer-Engine op layer
(fluid/core/te_ops.py:43-273): LayerNorm forward/backward with saved statistics and the
activation functions with their derivatives.  They dispatch to this library's kernels on CUDA and
to PyTorch on CPU."""
from __future__ import annotations

import torch

from . import norm


def te_layernorm_fwd(x, weight, bias, eps: float = 1e-5):
    y, _, _ = norm.norm_fwd(x.reshape(-1, x.shape[-1]), weight, bias, eps, "layernorm")
    return y.view_as(x)


def te_layernorm_fwd_with_stats(x, weight, bias, eps: float = 1e-5):
    y, mean, rstd = norm.norm_fwd(x.reshape(-1, x.shape[-1]), weight, bias, eps, "layernorm")
    return y.view_as(x), mean, rstd


def te_layernorm_bwd(dy, x, mean, rstd, weight, eps: float = 1e-5):
    """Uses the statistics saved by the forward pass (the reference's fallback recomputes the
    forward with a hard-coded eps, fluid/core/te_ops.py:134-140)."""
    dx, dw, db = norm.norm_bwd(dy.reshape(-1, x.shape[-1]), x.reshape(-1, x.shape[-1]), weight, mean, rstd,
                               "layernorm", True)
    return dx.view_as(x), dw, db


def te_gelu(x):
    return torch.nn.functional.gelu(x)


def te_silu(x):
    return torch.nn.functional.silu(x)


def te_dgelu(grad, x):
    xf = x.float()
    cdf = 0.5 * (1.0 + torch.erf(xf * 0.7071067811865476))
    pdf = torch.exp(-0.5 * xf * xf) * 0.3989422804014327
    return (grad.float() * (cdf + xf * pdf)).to(x.dtype)


def te_dsilu(grad, x):
    xf = x.float()
    s = torch.sigmoid(xf)
    return (grad.float() * s * (1.0 + xf * (1.0 - s))).to(x.dtype)


def create_te_dpa(*args, **kwargs):
    """Transformer Engine attention is not used: attention runs on this library's kernel."""
    return None


def create_te_linear(*args, **kwargs):
    """Transformer Engine linears are not used: projections are plain parameters."""
    return None
