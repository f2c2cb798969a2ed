"""Router: logits, top-k then softmax over the k winners, capacity dropping, slot assignment.

Semantics follow the reference router (fluid/moe/forward.py:393-466): the k largest logits are
selected first and soft-maxed among themselves in fp32; with a capacity ``cap = ceil(T*k/E*cf)``
each expert keeps its ``cap`` most probable tokens; every expert is then padded to exactly
``cap`` slots with not-routed tokens (ascending token id, probability 0), and the slots of an
expert are ordered by ascending token id.  Shapes are static, so nothing here synchronises
with the host.  The dropless variant keeps every routed pair and reports per-expert counts.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native


@dataclass
class RoutingPlan:
    sorted_indices: torch.Tensor     # [E*cap] int64: token id of every slot (expert-major)
    permuted_probs: torch.Tensor     # [E*cap] fp32: probability of every slot (0 for padding)
    slot_of_token: torch.Tensor      # [T, k] int32: slot of the j-th choice of token t, -1 = dropped
    tokens_per_expert: torch.Tensor  # [E] int32 (== cap in padded mode)
    routed_per_expert: torch.Tensor  # [E] int32 routed (non-padding) tokens after dropping
    routing_map: Optional[torch.Tensor]  # [T, E] bool after capacity dropping (None on the CUDA path)
    capacity: int


def expert_capacity(num_tokens: int, top_k: int, num_experts: int, capacity_factor: float) -> int:
    return int(math.ceil(num_tokens * top_k / num_experts * capacity_factor))


def router_logits(x: torch.Tensor, router_weight: torch.Tensor, router_dtype: torch.dtype) -> torch.Tensor:
    """``x[T,H] @ Wr[H,E]`` in ``router_dtype`` (weights detached: gradients are hand-written)."""
    w = router_weight.detach()
    if _native.use_native(x, w) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 \
            and router_dtype == torch.float32 and w.shape[1] % 8 == 0:
        # bf16 x bf16 products are exact in fp32, so the tensor-core GEMM with an fp32
        # accumulator equals casting both operands to fp32 first (up to summation order).
        from .gemm import grouped_gemm
        return grouped_gemm(x, w, b_layout="kn", out_dtype=torch.float32)
    if router_dtype != x.dtype:
        return x.to(router_dtype) @ w.to(router_dtype)
    return x @ w


def topk_softmax(logits: torch.Tensor, top_k: int, forced_idx: Optional[torch.Tensor] = None):
    """Top-k over experts, then softmax over the k selected logits in fp32.  ``forced_idx``
    (``[T, k]`` expert ids) replaces the selection and keeps the probabilities a function of the
    logits: used to replay one run's routing in another precision."""
    if forced_idx is not None:
        top_idx = forced_idx.to(device=logits.device, dtype=torch.int64)
        return top_idx, torch.softmax(logits.gather(1, top_idx).float(), dim=-1, dtype=torch.float32)
    if _native.use_native(logits) and logits.dtype == torch.float32 and hasattr(_native.lib(), "topk_softmax"):
        from . import elementwise
        return elementwise.topk_softmax(logits, top_k)
    top_logits, top_idx = torch.topk(logits, k=top_k, dim=-1)
    top_probs = torch.softmax(top_logits, dim=-1, dtype=torch.float32)
    return top_idx, top_probs


def build_padded_plan(top_idx: torch.Tensor, top_probs: torch.Tensor, num_experts: int,
                      capacity: int) -> RoutingPlan:
    """Capacity dropping + padded slot assignment with prefix sums (no sort, no host sync)."""
    T, k = top_idx.shape
    E = num_experts
    dev = top_idx.device
    assert capacity <= T, "capacity larger than the number of tokens is not supported"
    if _native.use_native(top_idx, top_probs) and k <= 16:
        from . import elementwise
        si, sp, sot, routed = elementwise.moe_plan(top_idx, top_probs, E, capacity)
        tpe = torch.full((E,), capacity, dtype=torch.int32, device=dev)
        return RoutingPlan(si, sp, sot, tpe, routed, None, capacity)
    probs = torch.zeros(T, E, dtype=torch.float32, device=dev).scatter(1, top_idx, top_probs.float())
    rmap = torch.zeros(T, E, dtype=torch.bool, device=dev).scatter(1, top_idx, True)
    if capacity < T:
        _, keep = torch.topk(probs, k=capacity, dim=0, sorted=False)
        cmask = torch.zeros(T, E, dtype=torch.bool, device=dev).scatter(0, keep, True)
        rmap = rmap & cmask
        probs = probs * rmap
    routed = rmap.sum(0, dtype=torch.int32)                       # [E]
    nonrouted_rank = torch.cumsum(~rmap, 0, dtype=torch.int32) - 1
    selected = rmap | ((~rmap) & (nonrouted_rank < (capacity - routed).unsqueeze(0)))
    pos = torch.cumsum(selected, 0, dtype=torch.int32) - 1        # slot inside the expert
    e_ids = torch.arange(E, device=dev, dtype=torch.int32).unsqueeze(0)
    flat = torch.where(selected, e_ids * capacity + pos, torch.full_like(pos, E * capacity)).long()
    tok = torch.arange(T, device=dev).unsqueeze(1).expand(T, E)
    sorted_indices = torch.zeros(E * capacity + 1, dtype=torch.int64, device=dev)
    sorted_indices.scatter_(0, flat.reshape(-1), tok.reshape(-1))
    sorted_indices = sorted_indices[:E * capacity]
    slot_probs = torch.zeros(E * capacity + 1, dtype=torch.float32, device=dev)
    slot_probs.scatter_(0, flat.reshape(-1), probs.reshape(-1))
    slot_probs = slot_probs[:E * capacity]
    # slot of the j-th choice of every token (-1 when that pair was dropped)
    slot_te = torch.where(rmap, e_ids * capacity + pos, torch.full_like(pos, -1))
    slot_of_token = slot_te.gather(1, top_idx).to(torch.int32)
    tpe = torch.full((E,), capacity, dtype=torch.int32, device=dev)
    return RoutingPlan(sorted_indices, slot_probs, slot_of_token, tpe, routed, rmap, capacity)


def build_dropless_plan(top_idx: torch.Tensor, top_probs: torch.Tensor, num_experts: int,
                        max_rows_per_expert: int, align: int = 1) -> RoutingPlan:
    """Keep every (token, expert) pair.  Expert e owns slots
    ``[e*max_rows, e*max_rows + count_e)`` of a buffer sized for the worst case
    (``max_rows_per_expert``, normally T), so shapes stay static; unused slots point at token 0
    with probability 0."""
    T, k = top_idx.shape
    E = num_experts
    dev = top_idx.device
    rmap = torch.zeros(T, E, dtype=torch.bool, device=dev).scatter(1, top_idx, True)
    probs = torch.zeros(T, E, dtype=torch.float32, device=dev).scatter(1, top_idx, top_probs.float())
    pos = torch.cumsum(rmap, 0, dtype=torch.int32) - 1
    counts = rmap.sum(0, dtype=torch.int32)
    e_ids = torch.arange(E, device=dev, dtype=torch.int32).unsqueeze(0)
    cap = max_rows_per_expert
    flat = torch.where(rmap, e_ids * cap + pos, torch.full_like(pos, E * cap)).long()
    tok = torch.arange(T, device=dev).unsqueeze(1).expand(T, E)
    sorted_indices = torch.zeros(E * cap + 1, dtype=torch.int64, device=dev)
    sorted_indices.scatter_(0, flat.reshape(-1), tok.reshape(-1))
    slot_probs = torch.zeros(E * cap + 1, dtype=torch.float32, device=dev)
    slot_probs.scatter_(0, flat.reshape(-1), probs.reshape(-1))
    slot_te = torch.where(rmap, e_ids * cap + pos, torch.full_like(pos, -1))
    return RoutingPlan(sorted_indices[:E * cap], slot_probs[:E * cap],
                       slot_te.gather(1, top_idx).to(torch.int32), counts, counts, rmap, cap)


def router_backward_logits(dprobs_slots: torch.Tensor, plan: RoutingPlan, top_idx: torch.Tensor,
                           top_probs: torch.Tensor, logits: torch.Tensor, num_experts: int,
                           aux_loss_coeff: float = 0.0, z_loss_coeff: float = 0.0,
                           tokens_per_expert_global: Optional[torch.Tensor] = None,
                           num_global_tokens: Optional[int] = None) -> torch.Tensor:
    """Gradient of the loss w.r.t. the router logits ``[T, E]`` (fp32).

    ``dprobs_slots`` is the gradient of every slot's probability.  The softmax backward runs over
    the k selected experts; the load-balancing (aux) loss contributes
    ``E * c / (k * T_g^2) * tokens_per_expert`` through the same softmax backward and the z-loss
    contributes ``2c/T * logsumexp(logits) * softmax(logits)`` (fluid/moe/backward.py:1461-1530).
    """
    T, k = top_idx.shape
    use_aux = aux_loss_coeff > 0.0 and tokens_per_expert_global is not None
    if (_native.use_native(dprobs_slots, top_idx) and hasattr(_native.lib(), "router_bwd")
            and plan.slot_of_token.dtype == torch.int32 and top_idx.dtype == torch.int64
            and (z_loss_coeff <= 0.0 or logits.dtype == torch.float32)):
        tg = float(num_global_tokens if num_global_tokens is not None else T)
        dlogits = torch.empty(T, num_experts, dtype=torch.float32, device=top_idx.device)
        dps = dprobs_slots.float().contiguous()
        tpe = tokens_per_expert_global.float().contiguous() if use_aux else None
        lg = logits.contiguous() if z_loss_coeff > 0.0 else None
        tp = top_probs.float().contiguous()
        _native.lib().router_bwd(dps.data_ptr(), plan.slot_of_token.contiguous().data_ptr(),
                                 top_idx.contiguous().data_ptr(), tp.data_ptr(),
                                 lg.data_ptr() if lg is not None else 0, tpe.data_ptr() if tpe is not None else 0,
                                 float(num_experts * aux_loss_coeff / (k * tg * tg)) if use_aux else 0.0,
                                 float(2.0 * z_loss_coeff / T) if z_loss_coeff > 0.0 else 0.0,
                                 T, k, num_experts, dlogits.data_ptr(), _native.stream_ptr())
        return dlogits
    slots = plan.slot_of_token.long()
    g = torch.where(slots >= 0, dprobs_slots.float()[slots.clamp(min=0)], torch.zeros((), device=slots.device))
    p = top_probs.float()
    if aux_loss_coeff > 0.0 and tokens_per_expert_global is not None:
        tg = float(num_global_tokens if num_global_tokens is not None else T)
        coef = num_experts * aux_loss_coeff / (k * tg * tg)
        g = g + coef * tokens_per_expert_global.float()[top_idx]
    dtop = p * (g - (p * g).sum(-1, keepdim=True))
    dlogits = torch.zeros(T, num_experts, dtype=torch.float32, device=top_idx.device).scatter(1, top_idx, dtop)
    if z_loss_coeff > 0.0:
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1, keepdim=True)
        dlogits = dlogits + (2.0 * z_loss_coeff / T) * lse * torch.softmax(lf, dim=-1)
    return dlogits
