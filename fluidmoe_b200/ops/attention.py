"""Causal grouped-query attention, forward and backward, on ``[s, b, heads, d]`` tensors.

The CUDA path is this library's flash-attention kernel (one pass over K/V per query tile, only
the log-sum-exp is saved); the PyTorch path below is the fp32 oracle and the CPU implementation.
The reference calls PyTorch SDPA or Transformer Engine here and differentiates through a saved
autograd sub-graph (fluid/attention/forward.py:280-329, fluid/layer/transformer.py:718-742); this
module exposes an explicit backward instead.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

from .. import _native


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float = None,
                  causal: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """q: [s, b, hq, d]; k, v: [s, b, hkv, d] (hq a multiple of hkv).  Returns ``(out, lse)``
    with out ``[s, b, hq, d]`` and lse ``[b, hq, s]`` fp32."""
    s, b, hq, d = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if q.is_cuda:
        return _sdpa_fwd(q, k, v, scale, causal)
    hkv = k.shape[2]
    rep = hq // hkv
    qf = q.float().permute(1, 2, 0, 3)                                   # [b, hq, s, d]
    kf = k.float().permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    sc = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(sc, dim=-1)
    p = torch.exp(sc - lse.unsqueeze(-1))
    out = torch.matmul(p, vf).permute(2, 0, 1, 3).contiguous().to(q.dtype)
    return out, lse


def attention_bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                  out: torch.Tensor, lse: torch.Tensor, scale: float = None, causal: bool = True):
    """Returns ``(dq, dk, dv)`` in the shapes of q, k, v."""
    s, b, hq, d = q.shape
    hkv = k.shape[2]
    rep = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if q.is_cuda:
        return _sdpa_bwd(dout, q, k, v, scale, causal, out, lse if (lse is not None and lse.dtype == torch.float32) else None)
    if lse is None:
        _, lse = attention_fwd(q, k, v, scale, causal)
    qf = q.float().permute(1, 2, 0, 3)
    kf = k.float().permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    do = dout.float().permute(1, 2, 0, 3)
    of = out.float().permute(1, 2, 0, 3)
    sc = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
    p = torch.exp(sc - lse.unsqueeze(-1))
    dv = torch.matmul(p.transpose(-1, -2), do)
    dp = torch.matmul(do, vf.transpose(-1, -2))
    delta = (do * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    dk = dk.view(b, hkv, rep, s, d).sum(2)
    dv = dv.view(b, hkv, rep, s, d).sum(2)
    to = lambda t, ref: t.permute(2, 0, 1, 3).contiguous().to(ref.dtype)  # noqa: E731
    return to(dq, q), to(dk, k), to(dv, v)


def native_forward(qkv: torch.Tensor, head_dim: int) -> bool:
    """Whether ``attention_fwd_packed`` will run this library's kernel on this input."""
    import os
    from . import flash
    return flash.supported(qkv, head_dim) and os.environ.get("FLUIDMOE_ATTN", "native") == "native"


def attention_fwd_packed(qkv: torch.Tensor, q_per_group: int, head_dim: int, scale: float = None, push=None):
    """Causal GQA attention on the packed projection buffer ``[s, b, G, (qpg + 2) * d]``.
    Returns ``(out [s, b, G*qpg, d], lse or None)``.  ``push``: see ``flash.flash_attn_fwd_packed``
    (only with the native kernel; the caller checks ``native_forward`` and ``flash.can_push``)."""
    from . import flash
    s, b, G, gs = qkv.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if native_forward(qkv, head_dim):
        return flash.flash_attn_fwd_packed(qkv, q_per_group, head_dim, scale, push=push)
    assert push is None, "the epilogue exchange needs the native attention kernel"
    heads = qkv.view(s, b, G, q_per_group + 2, head_dim)
    q = heads[:, :, :, :q_per_group].reshape(s, b, G * q_per_group, head_dim)
    return attention_fwd(q, heads[:, :, :, q_per_group], heads[:, :, :, q_per_group + 1], scale, True)


def attention_bwd_packed(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, lse, q_per_group: int,
                         head_dim: int, scale: float = None, wait=None) -> torch.Tensor:
    """Gradient of the packed projection buffer from the saved output (and log-sum-exp).
    ``FLUIDMOE_ATTN_BWD=native`` (default) selects this library's tcgen05 kernel, ``library`` the
    vendor attention backward."""
    import os
    from . import flash
    s, b, G, gs = qkv.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    have_lse = lse is not None and lse.dim() == 3 and lse.dtype == torch.float32
    if have_lse and flash.supported(qkv, head_dim) and os.environ.get("FLUIDMOE_ATTN_BWD", "native") == "native":
        return flash.flash_attn_bwd_packed(dout, qkv, out, lse, q_per_group, head_dim, scale, wait=wait)
    if wait is not None:
        wait["standalone"]()      # other back-ends cannot wait themselves
    qpg, d = q_per_group, head_dim
    heads = qkv.view(s, b, G, qpg + 2, d)
    q = heads[:, :, :, :qpg].reshape(s, b, G * qpg, d)
    dq, dk, dv = attention_bwd(dout.contiguous(), q, heads[:, :, :, qpg], heads[:, :, :, qpg + 1], out,
                               lse if have_lse else None, scale, True)
    dqkv = torch.empty_like(qkv)
    dh = dqkv.view(s, b, G, qpg + 2, d)
    dh[:, :, :, :qpg].copy_(dq.reshape(s, b, G, qpg, d))
    dh[:, :, :, qpg].copy_(dk)
    dh[:, :, :, qpg + 1].copy_(dv)
    return dqkv


# ---- library attention, used on CUDA where this library's own kernel does not apply ----
_CUDNN_DIRECT = {"ok": None}   # None = untested, True / False after the first attempt


def _sdpa_fwd(q, k, v, scale, causal):
    """Library forward.  When the fused cuDNN op is reachable directly it also yields the
    log-sum-exp, so the backward can run without recomputing the forward."""
    import torch.nn.functional as F
    hq, hkv = q.shape[2], k.shape[2]
    if _CUDNN_DIRECT["ok"] is not False and q.dtype in (torch.bfloat16, torch.float16):
        try:
            res = torch.ops.aten._scaled_dot_product_cudnn_attention(
                q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3), None, True, 0.0,
                causal, False, scale=scale)
            _CUDNN_DIRECT["ok"] = True
            lse = res[1]
            return res[0].permute(2, 0, 1, 3).contiguous(), lse.reshape(lse.shape[0], lse.shape[1], -1)
        except Exception:  # noqa: BLE001 - op unavailable for this shape / build
            if _CUDNN_DIRECT["ok"] is None:
                _CUDNN_DIRECT["ok"] = False
    out = F.scaled_dot_product_attention(q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3),
                                         v.permute(1, 2, 0, 3), is_causal=causal, scale=scale,
                                         enable_gqa=hq != hkv)
    return out.permute(2, 0, 1, 3).contiguous(), None


def _cudnn_bwd_direct(dout, q, k, v, out, lse, scale, causal):
    """Library backward from saved output and log-sum-exp ([b, h, s] fp32, natural log)."""
    s, b, hq, d = q.shape
    empty = torch.empty(0, device=q.device, dtype=torch.int32)
    seed = torch.zeros((), dtype=torch.int64, device=q.device)
    dq, dk, dv = torch.ops.aten._scaled_dot_product_cudnn_attention_backward(
        dout.permute(1, 2, 0, 3), q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3),
        out.permute(1, 2, 0, 3), lse.reshape(b, hq, s, 1).contiguous(), seed, seed, None, empty, empty,
        s, s, 0.0, causal, scale=scale)
    return dq.permute(2, 0, 1, 3), dk.permute(2, 0, 1, 3), dv.permute(2, 0, 1, 3)


def _sdpa_bwd(dout, q, k, v, scale, causal, out=None, lse=None):
    if out is not None and lse is not None and lse.dim() == 3 and _CUDNN_DIRECT["ok"] is not False:
        try:
            res = _cudnn_bwd_direct(dout, q, k, v, out, lse, scale, causal)
            _CUDNN_DIRECT["ok"] = True
            return res
        except Exception:  # noqa: BLE001
            _CUDNN_DIRECT["ok"] = False
    import torch.nn.functional as F
    hq, hkv = q.shape[2], k.shape[2]
    with torch.enable_grad():
        ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
        out = F.scaled_dot_product_attention(ql.permute(1, 2, 0, 3), kl.permute(1, 2, 0, 3),
                                             vl.permute(1, 2, 0, 3), is_causal=causal, scale=scale,
                                             enable_gqa=hq != hkv).permute(2, 0, 1, 3)
        return torch.autograd.grad(out, (ql, kl, vl), dout)
