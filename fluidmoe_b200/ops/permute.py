"""Token permute (gather rows into expert-major order) and un-permute (deterministic k-way sum).

The reference gathers with ``index_select`` / a Triton permute and sums with ``scatter_add_``
(atomics; fluid/moe/forward.py:446-461, fluid/layer/transformer.py:287-289).  Here the sum is a
gather over the (at most k) slots of every token, so the result does not depend on the order in
which contributions arrive.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native


def permute_rows(x: torch.Tensor, sorted_indices: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[s] = x[sorted_indices[s]]``."""
    if _native.use_native(x) and hasattr(_native.lib(), "gather_rows"):
        from . import elementwise
        res = elementwise.gather_rows(x, sorted_indices, out)
        if res is not None:
            return res
    res = x.index_select(0, sorted_indices.long())
    if out is not None:
        out.copy_(res)
        return out
    return res


def unpermute_reduce(rows: torch.Tensor, slot_of_token: torch.Tensor,
                     residual: Optional[torch.Tensor] = None, wait=None) -> torch.Tensor:
    """``out[t] = residual[t] + sum_j rows[slot_of_token[t, j]]`` (slots < 0 are skipped).
    ``wait``: see ``elementwise.unpermute_reduce`` (native kernel only; returns ``None`` when the
    native kernel cannot take this input, so that the caller can wait by other means)."""
    if _native.use_native(rows) and hasattr(_native.lib(), "unpermute_reduce"):
        from . import elementwise
        res = elementwise.unpermute_reduce(rows, slot_of_token, residual, wait)
        if res is not None:
            return res
    if wait is not None:
        return None
    T, k = slot_of_token.shape
    idx = slot_of_token.long()
    gathered = rows[idx.clamp(min=0)].float()                      # [T, k, H]
    gathered = gathered * (idx >= 0).unsqueeze(-1)
    out = gathered.sum(1)
    if residual is not None:
        out = out + residual.float()
    return out.to(rows.dtype)
