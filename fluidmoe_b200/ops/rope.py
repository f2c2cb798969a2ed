"""Rotary position embedding, non-interleaved ("rotate half") on the first ``rot_dim`` channels.

``freqs`` holds one angle per (position, channel) with the two halves equal, as produced by the
usual ``cat(f, f)`` construction; the transform is ``t * cos + rotate_half(t) * sin``
(fluid/layer/transformer.py:48-62).  The backward is the transposed rotation.  The packed
variant works in place on the ``[s, b, G, (q_per_group + 2) * d]`` QKV buffer and rotates the
query heads and the key head of every group, leaving the value head untouched.
"""
from __future__ import annotations

import torch

from .. import _native


def make_rope_freqs(seq_len: int, rot_dim: int, base: float = 10000.0, device=None) -> torch.Tensor:
    """Angles ``[seq, 1, 1, rot_dim]`` (fp32)."""
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
    pos = torch.arange(seq_len, dtype=torch.float32, device=device)
    f = torch.outer(pos, inv)
    return torch.cat([f, f], dim=-1).view(seq_len, 1, 1, rot_dim)


def _rotate(t: torch.Tensor, freqs: torch.Tensor, sign: float) -> torch.Tensor:
    rot = freqs.shape[-1]
    tr = t[..., :rot].float()
    cos, sin = torch.cos(freqs.float()), torch.sin(freqs.float()) * sign
    x1, x2 = tr.chunk(2, dim=-1)
    if sign > 0:
        out = tr * cos + torch.cat((-x2, x1), dim=-1) * sin
    else:
        # transpose of the forward map: d1' = d1 cos + d2 sin(f2), d2' = d2 cos - d1 sin(f1)
        s1, s2 = (torch.sin(freqs.float())).chunk(2, dim=-1)
        c1, c2 = torch.cos(freqs.float()).chunk(2, dim=-1)
        out = torch.cat((x1 * c1 + x2 * s2, x2 * c2 - x1 * s1), dim=-1)
    out = out.to(t.dtype)
    if rot == t.shape[-1]:
        return out
    return torch.cat((out, t[..., rot:]), dim=-1)


def apply_rope(t: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """t: [s, b, h, d]; freqs: [s, 1, 1, rot_dim]."""
    return _rotate(t, freqs, 1.0)


def apply_rope_bwd(dt: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    return _rotate(dt, freqs, -1.0)


def rope_packed_(qkv: torch.Tensor, freqs: torch.Tensor, q_per_group: int, head_dim: int,
                 backward: bool = False, wait=None) -> torch.Tensor:
    """In place on ``qkv [s, b, G, (q_per_group + 2) * d]``: rotate q heads and the k head.
    ``wait`` (``dict(flags, n, expected, wait_ns, timeout_ns, status, standalone)``): ``qkv`` is still
    being filled by peers; the native kernel waits for their arrival counters itself, any other path
    calls ``wait["standalone"]()`` first."""
    s, b, G, gs = qkv.shape
    if _native.use_native(qkv) and hasattr(_native.lib(), "rope_packed"):
        from . import elementwise
        res = elementwise.rope_packed_(qkv, freqs, q_per_group, head_dim, backward, wait)
        if res is not None:
            return res
    if wait is not None:
        wait["standalone"]()
    heads = qkv.view(s, b, G, q_per_group + 2, head_dim)
    part = heads[..., : q_per_group + 1, :].reshape(s, b, G * (q_per_group + 1), head_dim)
    fn = apply_rope_bwd if backward else apply_rope
    heads[..., : q_per_group + 1, :] = fn(part, freqs).view(s, b, G, q_per_group + 1, head_dim)
    return qkv
