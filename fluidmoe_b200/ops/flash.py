"""Front-end of the tcgen05 flash-attention kernel (packed QKV layout, head dim 128)."""
from __future__ import annotations

import torch

from .. import _native
from .gemm import status_buffer

import os

LAUNCHES = 0
VERSION = int(os.environ.get("FLUIDMOE_FLASH_VERSION", "2"))
BWD_VERSION = int(os.environ.get("FLUIDMOE_FLASH_BWD_VERSION", "2"))


def supported(qkv: torch.Tensor, head_dim: int) -> bool:
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim == 128 and qkv.is_contiguous()
            and _native.available() and hasattr(_native.lib(), "flash_attn_fwd"))


def can_push(qkv: torch.Tensor, rows_per_rank: int, version: int = 0) -> bool:
    """Whether the forward kernel can do the HP -> SP exchange in its epilogue for this input."""
    return (version or VERSION) == 2 and qkv.shape[1] == 1 and rows_per_rank > 0 and rows_per_rank % 128 == 0


def flash_attn_fwd_packed(qkv: torch.Tensor, q_per_group: int, head_dim: int, scale: float, version: int = 0,
                          push=None):
    """qkv: [s, b, G, (qpg + 2) * d] -> (out [s, b, G*qpg, d], lse [b, G*qpg, s]).

    ``push`` (``dict(dst_table, flags_table, me, P, rows_per_rank, row_blocks)``): every output row is
    also stored into the sequence owner's buffer and the owner's arrival counter is raised, which
    replaces the separate HP -> SP push (fluid/attention/forward.py:435-476)."""
    global LAUNCHES
    s, b, G, gs = qkv.shape
    hq = G * q_per_group
    out = torch.empty(s, b, hq, head_dim, dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty(b, hq, s, dtype=torch.float32, device=qkv.device)
    LAUNCHES += 1
    if push is None:
        _native.lib().flash_attn_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), s, b, G, q_per_group,
                                     head_dim, float(scale), 0, status_buffer(qkv.device).data_ptr(),
                                     version or VERSION, _native.stream_ptr())
    else:
        _native.lib().flash_attn_fwd_push(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), s, b, G, q_per_group,
                                          head_dim, float(scale), 0, status_buffer(qkv.device).data_ptr(),
                                          version or VERSION, push["dst_table"], push["flags_table"],
                                          push["me"], push["P"], push["rows_per_rank"], push["row_blocks"],
                                          _native.stream_ptr())
    return out, lse


def flash_attn_bwd_packed(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                          q_per_group: int, head_dim: int, scale: float, version: int = 0,
                          head_split=None, wait=None) -> torch.Tensor:
    """Gradient of the packed projection buffer, ``[s, b, G, (qpg + 2) * d]`` (dq heads, dk, dv per
    KV group), from the saved output and log-sum-exp.  ``wait`` (``dict(flags, n, expected, wait_ns)``,
    addresses as ints): per-source arrival counters of ``dout`` that the first kernel waits for."""
    global LAUNCHES
    s, b, G, gs = qkv.shape
    hq = G * q_per_group
    dout = dout.contiguous()
    delta = torch.empty(b, hq, s, dtype=torch.float32, device=qkv.device)
    dq_accum = torch.zeros(s, b, hq, head_dim, dtype=torch.float32, device=qkv.device)
    dqkv = torch.empty_like(qkv)
    ver = version or BWD_VERSION
    # Causal work per CTA is triangular; with few (K/V block, KV head) pairs the query heads of a group
    # are split over several CTAs, which then add their dK / dV parts into an fp32 buffer.
    hsplit = 1
    if ver == 2 and head_split is not False:
        ctas = ((s + 127) // 128) * G * b
        hsplit = head_split if head_split else 1
        if not head_split:
            while hsplit * 2 <= q_per_group and q_per_group % (hsplit * 2) == 0 and ctas * hsplit < 4 * 148:
                hsplit *= 2
    dkv = torch.zeros(s, b, G, 2, head_dim, dtype=torch.float32, device=qkv.device) if hsplit > 1 else None
    LAUNCHES += 3 + (1 if hsplit > 1 else 0)
    args = (qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), delta.data_ptr(),
            dq_accum.data_ptr(), dqkv.data_ptr(), s, b, G, q_per_group, head_dim, float(scale),
            0, status_buffer(qkv.device).data_ptr(), ver, dkv.data_ptr() if dkv is not None else 0, hsplit)
    if wait is None:
        _native.lib().flash_attn_bwd(*args, _native.stream_ptr())
    else:
        # `dout` is still being filled by peers: the first kernel waits for their arrival counters
        _native.lib().flash_attn_bwd_gated(*args, wait["flags"], wait["n"], wait["expected"], wait["wait_ns"],
                                           _native.stream_ptr())
    return dqkv
