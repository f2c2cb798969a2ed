"""One MoE transformer block as a single autograd node with a hand-written backward.

    x -> norm1 -> QKV (+SP->HP) -> RoPE -> causal GQA attention -> (HP->SP+) out-proj -> +x
      -> norm2 -> router -> dispatch + FC1 -> FC2 + combine -> un-permute (+shared experts) -> +h

The backward walks the four communication regions in reverse (``moe_combine``, ``moe_dispatch``,
``attn_proj``, ``attn_qkv``), computes input gradients on the critical path and hands every weight
gradient to the backward scheduler, which runs it inside a later communication window
(fluid/layer/transformer.py:65-810 of the reference).  Tensors are ``[seq, batch, hidden]``.

Differences from the reference layer that the target configurations need: RMSNorm as well as
LayerNorm, gated (SwiGLU) experts, shared experts, fp32 routing probabilities end to end, an
explicit attention backward (no saved autograd sub-graph) and a CPU/gloo execution path.
"""
from __future__ import annotations

import math
import os
from typing import Callable, Optional, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import attention as attn_ops
from ..ops import gemm, norm, permute, rope, router as router_ops
from ..parallel import comm
from ..parallel.scheduler import get_backward_scheduler
from ..parallel.schedule import MultiCardOverlapContext
from ..utils.nvtx import nvtx_range
from . import attention as attn_mod
from . import moe as moe_mod
from . import moe_dropless


def _activation_name(fn: Union[str, Callable, None]) -> str:
    if fn is None:
        return "gelu"
    if isinstance(fn, str):
        name = fn.lower()
    else:
        name = getattr(fn, "__name__", "gelu").lower()
    for key in ("swiglu", "silu", "gelu"):
        if key in name:
            return key
    if "swish" in name:
        return "silu"
    raise ValueError(f"unsupported activation {fn!r}")


class LayerRuntime:
    """Per-layer static configuration and lazily built plans, passed through the autograd node."""

    def __init__(self, layer: "TransformerLayer"):
        self.layer = layer
        self.ep_plan: Optional[moe_mod.EPPlan] = None
        self.cp_plan: Optional[attn_mod.CPPlan] = None
        self.sig = None
        self.grad_enabled = True     # grad mode of the current forward call (set by the module)

    def ensure(self, x: torch.Tensor) -> None:
        L = self.layer
        gen = L.fused_ctx.generation if L.fused_ctx is not None else 0
        sig = (x.shape[0], x.shape[1], x.dtype, x.device, gen)
        if sig == self.sig:
            return
        self.sig = sig
        s_loc, b, H = x.shape
        self.ep_plan = moe_mod.EPPlan(s_loc * b, H, L.num_experts, L.top_k, L.ep_group,
                                      L.capacity_factor if not L.dropless else 1.0, x.dtype, x.device,
                                      L.moe_overlap_ctx)
        self.cp_plan = attn_mod.CPPlan(s_loc, b, H, L.num_heads, L.num_kv_heads, L.head_dim,
                                       L.cp_group, x.dtype, x.device, L.attn_overlap_ctx)
        self.ep_plan.layer_id = self.cp_plan.layer_id = L.layer_id
        L._moe_chunk_config = moe_mod.build_moe_chunk_config(
            L.moe_combine_chunks, L.moe_dispatch_chunks, self.ep_plan.num_local_experts,
            self.ep_plan.expert_capacity)
        if L.fused_ctx is not None:
            L.fused_ctx.prepare(self.ep_plan, self.cp_plan, L)
            # a new shape released every layer's buffers: remember the generation now current
            self.sig = sig[:4] + (L.fused_ctx.generation,)


class TransformerLayerFunction(torch.autograd.Function):
    """Forward and backward of one block.  Weight gradients are never returned to autograd: they
    are produced by scheduler tasks (into ``param.grad``, or into ``param.main_grad`` when the
    parameter is registered in a flat gradient buffer)."""

    @staticmethod
    def forward(ctx, x, ln1_w, ln1_b, ln2_w, ln2_b, qkv_w, proj_w, router_w, w1, w2,
                shared_w1, shared_w2, rotary, rt: LayerRuntime):
        L = rt.layer
        rt.ensure(x)
        ep, cp = rt.ep_plan, rt.cp_plan
        s_loc, b, H = x.shape
        T = s_loc * b
        x2 = x.reshape(T, H)
        # ``needs_input_grad`` ignores torch.no_grad(); the module records the grad mode it was
        # called in, so that an inference pass neither keeps activations nor the FC1 pre-activation
        needs_grad = any(ctx.needs_input_grad) and rt.grad_enabled
        act = L.activation
        mode_attn = L.resolve_mode(cp.cp_size, attention=True, cp_plan=cp)
        mode_moe = L.resolve_mode(ep.ep_size)
        fused = L.fused_ctx
        uses_fused = fused is not None and (("fused" == mode_attn and L.has_attention) or
                                            ("fused" == mode_moe and L.has_moe and ep.ep_size > 1))
        if uses_fused:
            fused.layer_forward_begin(ep, needs_grad)

        # ---- attention half ----
        mean1 = rstd1 = ln1_out = qkv_full = attn_out = lse = attn_in_full = None
        if L.has_attention:
            with nvtx_range("ln1"):
                ln1_out, mean1, rstd1 = norm.norm_fwd(x2, ln1_w, ln1_b, L.norm_eps, L.norm_type)
            # device-initiated transport: the first kernel that reads a buffer peers are filling waits
            # for their arrival counters itself (here RoPE), no stand-alone wait kernel in between
            defer = mode_attn == "fused" and cp.cp_size > 1 and rotary is not None
            with nvtx_range("qkv_sp2hp"):
                qkv_full = attn_mod.qkv_projection_forward(ln1_out, qkv_w, cp, mode_attn, fused, defer_wait=defer)
            if rotary is not None:
                rope.rope_packed_(qkv_full, rotary, cp.q_per_group, cp.head_dim,
                                  wait=fused.take_pending_wait() if defer else None)
                if defer:
                    fused.finish_pending_wait()
            G, qpg, d = cp.groups_per_rank, cp.q_per_group, cp.head_dim
            # with the device-initiated transport the attention kernel's epilogue stores every output
            # row at its sequence owner as well (when the shape allows), so no push kernel follows
            push = (fused.attention_push_args(cp, qkv_full)
                    if mode_attn == "fused" and cp.cp_size > 1 and L.attention_epilogue_push else None)
            with nvtx_range("attention"):
                attn_out, lse = attn_ops.attention_fwd_packed(qkv_full, qpg, d, 1.0 / math.sqrt(d), push=push)
            with nvtx_range("hp2sp_outproj"):
                h1, attn_in_full = attn_mod.output_projection_forward(attn_out, proj_w, cp, mode_attn, fused,
                                                                      residual=x2, pushed=push is not None)
        else:
            h1 = x2

        # ---- MoE half ----
        mean2 = rstd2 = ln2_out = top_idx = top_probs = logits = rplan = st = None
        sh_pre = sh_act = None
        if not L.has_moe:
            out = h1
        else:
            with nvtx_range("ln2"):
                ln2_out, mean2, rstd2 = norm.norm_fwd(h1, ln2_w, ln2_b, L.norm_eps, L.norm_type)
            save_pre = needs_grad and not L.recompute_fc1
            if L.dropless:
                fused_dropless = mode_moe == "fused" and ep.ep_size > 1
                mode_moe = "dropless_fused" if fused_dropless else "dropless"
                logits = router_ops.router_logits(ln2_out, router_w, L.router_dtype)
                if L.router_logit_bias is not None:
                    logits = logits + L.router_logit_bias
                top_idx, top_probs = router_ops.topk_softmax(logits, L.top_k, L.forced_top_idx)
                with nvtx_range("dropless_moe"):
                    if fused_dropless:
                        # device-initiated: counts exchanged by peer stores, no host read anywhere
                        from ..parallel.fused_dropless import build_device_plan
                        rplan = build_device_plan(top_idx, top_probs, L.num_experts)
                        combined, st = fused.dropless.forward(fused._buf(ep), ep, rplan, ln2_out, w1, w2, act,
                                                              save_pre, needs_grad)
                    else:
                        rplan = moe_dropless.build_plan(top_idx, top_probs, L.num_experts, L.ep_group)
                        combined, st = moe_dropless.forward(rplan, ln2_out, w1, w2, act, L.ep_group, save_pre)
            else:
                gather = not (mode_moe == "fused" and ep.ep_size > 1)
                (permuted, probs, sorted_idx, _tpe, top_idx, top_probs, logits, _rmap, rplan) = \
                    moe_mod.router_forward(ln2_out, router_w, L.num_experts, L.top_k, L.ep_group,
                                           L.capacity_factor, ep, L.router_dtype, gather_tokens=gather,
                                           forced_top_idx=L.forced_top_idx, logit_bias=L.router_logit_bias)
                with nvtx_range("dispatch_fc1"):
                    st = moe_mod.dispatch_fc1_forward(ep, permuted, probs, w1, act, mode_moe, save_pre=save_pre,
                                                      fused_ctx=fused, hidden_states=ln2_out,
                                                      sorted_indices=sorted_idx)
                with nvtx_range("fc2_combine"):
                    combined = moe_mod.fc2_combine_forward(ep, st, w2, mode_moe, fused)
            if needs_grad and L.recompute_fc1:
                # the FC1 pre-activation is rebuilt in the backward pass from the saved tokens
                groups = (dict(group_rows=rplan.group_rows, group_offs=rplan.group_offs) if L.dropless else
                          dict(uniform_rows=(ep.ep_size if ep.ep_size > 1 else 1) * ep.expert_capacity))
                st.set_recompute(lambda st=st, w1=w1, groups=groups: gemm.grouped_gemm(
                    st.tokens_em, w1.detach(), b_layout="kn", **groups))
            residual = h1
            if shared_w1 is not None:
                sh_act, sh_pre = gemm.grouped_gemm_act(ln2_out, shared_w1.unsqueeze(0), None,
                                                       activation=L.shared_activation, save_pre=needs_grad)
                residual = gemm.gemm_nn(sh_act, shared_w2, out=h1.clone(), accumulate=True)
            with nvtx_range("unpermute"):
                if mode_moe == "dropless_fused":
                    out = fused.dropless.unpermute(fused._buf(ep), rplan, combined, residual, "combined")
                elif mode_moe == "fused" and ep.ep_size > 1:
                    out = fused.unpermute(ep, combined, rplan.slot_of_token, residual)
                else:
                    out = permute.unpermute_reduce(combined, rplan.slot_of_token, residual)

        if needs_grad:
            ctx.rt = rt
            ctx.modes = (mode_attn, mode_moe)
            ctx.uses_fused = uses_fused
            ctx.has_rotary = rotary is not None
            ctx.has_shared = shared_w1 is not None
            ctx.rplan = rplan
            ctx.st = st
            ctx.params = (ln1_w, ln1_b, ln2_w, ln2_b, qkv_w, proj_w, router_w, w1, w2, shared_w1, shared_w2)
            ph = x2      # placeholder for tensors a skipped half or option does not produce
            opt = lambda t: t if t is not None else ph   # noqa: E731
            ctx.save_for_backward(x2, opt(mean1 if mean1 is not None else rstd1), opt(rstd1), opt(ln1_out),
                                  opt(qkv_full), opt(attn_out), opt(lse), opt(attn_in_full), h1,
                                  opt(mean2 if mean2 is not None else rstd2), opt(rstd2), opt(ln2_out),
                                  opt(top_idx), opt(top_probs), opt(logits), opt(rotary), opt(sh_pre), opt(sh_act))
            ctx.has_lse = lse is not None
        return out.view(s_loc, b, H)

    @staticmethod
    def backward(ctx, dy):
        rt: LayerRuntime = ctx.rt
        L = rt.layer
        ep, cp = rt.ep_plan, rt.cp_plan
        mode_attn, mode_moe = ctx.modes
        fused = L.fused_ctx
        sched = get_backward_scheduler()
        (x2, mean1, rstd1, ln1_out, qkv_full, attn_out, lse, attn_in_full, h1, mean2, rstd2, ln2_out,
         top_idx, top_probs, logits, rotary, sh_pre, sh_act) = ctx.saved_tensors
        (ln1_w, ln1_b, ln2_w, ln2_b, qkv_w, proj_w, router_w, w1, w2, shared_w1, shared_w2) = ctx.params
        rplan, st = ctx.rplan, ctx.st
        act = L.activation
        lid = L.layer_id
        is_ln = L.norm_type == "layernorm"
        T, H = x2.shape
        s_loc = cp.seq_local
        b = cp.batch
        dy2 = dy.reshape(T, H).contiguous()
        P = ep.ep_size
        nle, cap = ep.num_local_experts, ep.expert_capacity
        cfg = L._moe_chunk_config

        if not L.has_moe:
            dh1 = dy2
        elif mode_moe == "dropless_fused":
            # variable-split path on the device-initiated transport: same regions as the padded
            # path, row ranges and arrival thresholds come from the device-side plan
            dl, db = fused.dropless, fused._buf(ep)
            with nvtx_range("bwd_moe_combine"):
                sched.begin_region("moe_combine")
                try:
                    dfc2_em, dpre_em, dprobs_em = dl.combine_fc2_backward(db, ep, rplan, dy2, st, w2, act)
                finally:
                    sched.end_region()
            w1_late = getattr(w1, "_fused_adam", None) is not None
            if not w1_late:
                moe_dropless.register_dw_tasks(rplan, st, dfc2_em, dpre_em, w1, w2, lid, f"layer{lid}.moe")
            else:
                moe_dropless.register_dw_tasks(rplan, st, dfc2_em, dpre_em, w1, w2, lid, f"layer{lid}.moe", which="w2")
            with nvtx_range("bwd_moe_dispatch"):
                sched.begin_region("moe_dispatch")
                try:
                    dperm = dl.fc1_dispatch_backward(db, ep, dpre_em, w1, dprobs_em)
                finally:
                    sched.end_region()
                dl.wait_rows(db, "dperm")
                tpe_global = None
                if L.aux_loss_coeff > 0.0:
                    tpe_global = rplan.routed_per_expert.float()
                    if cp.cp_size > 1:
                        dist.all_reduce(tpe_global, group=cp.group)
                dlogits = router_ops.router_backward_logits(
                    db.dprobs_perm.local, rplan, top_idx, top_probs, logits, L.num_experts, L.aux_loss_coeff,
                    L.z_loss_coeff, tpe_global, T * cp.cp_size)
                d_ln2_router = (dlogits.to(router_w.dtype) @ router_w.detach().t()).to(dy2.dtype)
                ln2_for_dw = ln2_out
                sched.register_dw_task(f"layer{lid}.router", lid,
                                       lambda: (ln2_for_dw.float().t() @ dlogits).to(torch.float32), router_w)
                d_ln2 = dl.unpermute(db, rplan, dperm, d_ln2_router, "dperm", waited=True)
            if w1_late:
                moe_dropless.register_dw_tasks(rplan, st, dfc2_em, dpre_em, w1, w2, lid, f"layer{lid}.moe", which="w1")
        elif mode_moe == "dropless":
            # variable-split path: all-to-all-v in, grouped GEMMs over device-sized groups, all-to-all-v out
            with nvtx_range("bwd_dropless_moe"):
                grad_combined = permute.permute_rows(dy2, rplan.sorted_indices)
                dfc2_em, dpre_em, dprobs_perm, dperm = moe_dropless.backward(rplan, grad_combined, st, w1, w2,
                                                                             act, L.ep_group)
            moe_dropless.register_dw_tasks(rplan, st, dfc2_em, dpre_em, w1, w2, lid, f"layer{lid}.moe")
            tpe_global = None
            if L.aux_loss_coeff > 0.0:
                tpe_global = rplan.routed_per_expert.float()
                if cp.cp_size > 1:
                    dist.all_reduce(tpe_global, group=cp.group)
            dlogits = router_ops.router_backward_logits(
                dprobs_perm, rplan, top_idx, top_probs, logits, L.num_experts, L.aux_loss_coeff,
                L.z_loss_coeff, tpe_global, T * cp.cp_size)
            d_ln2_router = (dlogits.to(router_w.dtype) @ router_w.detach().t()).to(dy2.dtype)
            ln2_for_dw = ln2_out
            sched.register_dw_task(f"layer{lid}.router", lid,
                                   lambda: (ln2_for_dw.float().t() @ dlogits).to(torch.float32), router_w)
            d_ln2 = permute.unpermute_reduce(dperm, rplan.slot_of_token, d_ln2_router)
        else:
            # ---- R1: combine gradient -> FC2 dX + activation backward ----
            with nvtx_range("bwd_moe_combine"):
                if mode_moe == "fused" and P > 1:
                    grad_combined = None
                else:
                    grad_combined = permute.permute_rows(dy2, rplan.sorted_indices)
                dfc2_em, dpre_em, dprobs_em = moe_mod.combine_fc2_backward(
                    ep, grad_combined, st, w2, act, cfg["moe_combine"].num_chunks, mode_moe,
                    fused_ctx=_FusedBwd(fused, dy2, rplan) if (mode_moe == "fused" and P > 1) else None)
            # w1 is still needed by the FC1 dX GEMM of R2: when its optimizer runs in the
            # weight-gradient epilogue the task may only be queued after R2
            w1_late = getattr(w1, "_fused_adam", None) is not None
            moe_mod.register_moe_dw_tasks(ep, st, dfc2_em, dpre_em, w1, w2, lid, f"layer{lid}.moe",
                                          which="w2" if w1_late else "both")

            fused_moe = mode_moe == "fused" and P > 1

            def router_backward(dprobs_perm):
                """Routing-probability gradient (permuted order, on the token owner) -> gradient of
                the router input; queues the router weight gradient."""
                tpe_global = None
                if L.aux_loss_coeff > 0.0:
                    tpe_global = rplan.routed_per_expert.float()
                    if cp.cp_size > 1:
                        dist.all_reduce(tpe_global, group=cp.group)
                dlogits = router_ops.router_backward_logits(
                    dprobs_perm, rplan, top_idx, top_probs, logits, L.num_experts, L.aux_loss_coeff,
                    L.z_loss_coeff, tpe_global, T * cp.cp_size)
                d_router = (dlogits.to(router_w.dtype) @ router_w.detach().t()).to(dy2.dtype)
                ln2_for_dw = ln2_out

                def router_dw():
                    return (ln2_for_dw.float().t() @ dlogits).to(torch.float32)
                sched.register_dw_task(f"layer{lid}.router", lid, router_dw, router_w)
                return d_router

            # ---- routing-probability gradient back to the token owners, router backward ----
            # Device-initiated transport: the probability gradient of a row rides with the row's
            # dispatch gradient in the FC1 input-gradient epilogue (region moe_dispatch), so the
            # router backward runs after that exchange.  Other transports: a small all-to-all now.
            d_ln2_router = None
            if not fused_moe:
                with nvtx_range("bwd_router"):
                    if P > 1:
                        send = moe_mod.expert_to_rank_major(dprobs_em, P, nle, cap).contiguous()
                        dprobs_perm = comm.all_to_all(send, ep.group)
                    else:
                        dprobs_perm = dprobs_em
                    d_ln2_router = router_backward(dprobs_perm)

            # ---- R2: FC1 dX -> dispatch gradient -> token order ----
            with nvtx_range("bwd_moe_dispatch"):
                dperm = moe_mod.fc1_dispatch_backward(ep, dpre_em, w1, cfg["moe_dispatch"].num_chunks, mode_moe,
                                                      fused_ctx=fused, dprobs_em=dprobs_em if fused_moe else None)
                if fused_moe:
                    with nvtx_range("bwd_router"):
                        d_ln2_router = router_backward(fused.wait_dispatch_grad(ep))
                    d_ln2 = fused.unpermute(ep, dperm, rplan.slot_of_token, d_ln2_router, waited=True)
                else:
                    d_ln2 = permute.unpermute_reduce(dperm, rplan.slot_of_token, d_ln2_router)
            if w1_late:
                moe_mod.register_moe_dw_tasks(ep, st, dfc2_em, dpre_em, w1, w2, lid, f"layer{lid}.moe", which="w1")

        # ---- shared experts (dense, local) ----
        if ctx.has_shared and L.has_moe:
            dsh_pre, _ = gemm.grouped_gemm_dact(dy2, shared_w2.unsqueeze(0), sh_pre, None,
                                                activation=L.shared_activation)
            d_ln2 = gemm.gemm_nt(dsh_pre, shared_w1, out=d_ln2, accumulate=True)
            attn_mod._register_dense_dw(f"layer{lid}.shared_w2", lid, sh_act, dy2, shared_w2, transpose_out=True)
            attn_mod._register_dense_dw(f"layer{lid}.shared_w1", lid, ln2_out, dsh_pre, shared_w1, transpose_out=True)

        # ---- norm2 backward (+ residual gradient) ----
        if L.has_moe:
            dh1, dln2_w, dln2_b = norm.norm_bwd(d_ln2, h1, ln2_w, mean2 if is_ln else None, rstd2,
                                                L.norm_type, is_ln, residual_grad=dy2)
            sched.register_dw_task(f"layer{lid}.ln2_w", lid, lambda: dln2_w, ln2_w)
            if is_ln:
                sched.register_dw_task(f"layer{lid}.ln2_b", lid, lambda: dln2_b, ln2_b)
        if not L.has_attention:
            ctx.st = ctx.rplan = None
            if ctx.uses_fused:
                fused.layer_backward_end(ep)
            return (dh1.view(s_loc, b, H),) + (None,) * 13

        # ---- R3: out-proj dX -> SP->HP ----
        attn_mod.output_projection_register_dw(lid, attn_in_full, dh1, proj_w)
        defer = mode_attn == "fused" and cp.cp_size > 1     # the attention backward waits for the exchange itself
        with nvtx_range("bwd_attn_proj"):
            d_attn = attn_mod.outproj_sp2hp_backward(dh1, proj_w, cp, L.attn_proj_chunks, mode_attn, fused,
                                                     defer_wait=defer)

        # ---- attention backward (+ RoPE backward), packed per KV group ----
        with nvtx_range("bwd_attention"):
            G, qpg, d = cp.groups_per_rank, cp.q_per_group, cp.head_dim
            dqkv_hp = attn_ops.attention_bwd_packed(d_attn, qkv_full, attn_out,
                                                    lse if ctx.has_lse else None, qpg, d,
                                                    1.0 / math.sqrt(d),
                                                    wait=fused.take_pending_wait() if defer else None)
            if defer:
                fused.finish_pending_wait()
            if ctx.has_rotary:
                rope.rope_packed_(dqkv_hp, rotary, qpg, d, backward=True)

        # ---- R4: HP->SP -> QKV dX ----
        with nvtx_range("bwd_attn_qkv"):
            d_ln1, dqkv_sp = attn_mod.hp2sp_qkv_backward(dqkv_hp, qkv_w, cp, L.attn_qkv_chunks, mode_attn, fused)
        attn_mod.register_qkv_dw(lid, ln1_out, dqkv_sp, qkv_w)

        # ---- norm1 backward (+ residual gradient) ----
        dx, dln1_w, dln1_b = norm.norm_bwd(d_ln1, x2, ln1_w, mean1 if is_ln else None, rstd1,
                                           L.norm_type, is_ln, residual_grad=dh1)
        sched.register_dw_task(f"layer{lid}.ln1_w", lid, lambda: dln1_w, ln1_w)
        if is_ln:
            sched.register_dw_task(f"layer{lid}.ln1_b", lid, lambda: dln1_b, ln1_b)
        ctx.st = ctx.rplan = None
        if ctx.uses_fused:
            fused.layer_backward_end(ep)
        return (dx.view(s_loc, b, H),) + (None,) * 13


class _FusedBwd:
    """Adapter giving the fused R1 path access to the un-permuted output gradient."""

    def __init__(self, fused, dy2, rplan):
        self.fused, self.dy2, self.rplan = fused, dy2, rplan

    def combine_fc2_backward(self, plan, grad_combined, state, w2, activation):
        return self.fused.combine_fc2_backward(plan, self.dy2, self.rplan, state, w2, activation)


class TransformerLayer(nn.Module):
    """Standalone MoE transformer block.

    Constructor arguments follow the reference layer (fluid/layer/transformer.py:836-862);
    ``norm_type``, ``num_shared_experts``, ``shared_ffn_hidden_size``, ``comm_mode``, ``norm_eps``
    and ``parallel_ctx`` are additions.  ``comm_mode``: ``auto`` (fused kernels when a symmetric
    heap is attached, else pairwise overlap), ``a2a``, ``p2p`` or ``fused``.
    """

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, ffn_hidden_size: int,
                 num_experts: int, top_k: int, cp_group=None, ep_group=None, layer_id: int = 0,
                 moe_combine_chunks: int = 1, moe_dispatch_chunks: int = 1, attn_proj_chunks: int = 1,
                 attn_qkv_chunks: int = 1, activation_func=None, capacity_factor: float = 1.0,
                 init_std: float = 0.02, output_init_std: Optional[float] = None,
                 dtype: torch.dtype = torch.bfloat16, device=None,
                 router_dtype: torch.dtype = torch.bfloat16, aux_loss_coeff: float = 0.0,
                 z_loss_coeff: float = 0.0, *, norm_type: str = "layernorm", norm_eps: float = 1e-5,
                 num_shared_experts: int = 0, shared_ffn_hidden_size: Optional[int] = None,
                 comm_mode: str = "auto", parallel_ctx=None, has_attention: bool = True, has_moe: bool = True,
                 recompute_fc1: bool = False):
        super().__init__()
        assert has_attention or has_moe
        # Either half can be switched off (its parameters stay in the state dict and receive no
        # gradient): the block benchmarks time the MoE half and the attention half on their own.
        self.has_attention, self.has_moe = bool(has_attention), bool(has_moe)
        # Drop the FC1 pre-activation after the forward pass and rebuild it in the backward pass
        # (one more FC1 GEMM per layer for [rows, F or 2F] less saved memory).
        self.recompute_fc1 = bool(recompute_fc1)
        # HP -> SP exchange inside the attention kernel's epilogue (device-initiated transport only)
        self.attention_epilogue_push = os.environ.get("FLUIDMOE_ATTN_EPILOGUE_PUSH", "1") == "1"
        self.router_logit_bias = None   # optional fp32 [E] prior added to the router logits (set_router_bias)
        if parallel_ctx is not None:
            cp_group = cp_group if cp_group is not None else parallel_ctx.cp_group
            ep_group = ep_group if ep_group is not None else parallel_ctx.ep_group
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
                else torch.device("cpu")
        device = torch.device(device)
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.ffn_hidden_size, self.num_experts, self.top_k = ffn_hidden_size, num_experts, top_k
        self.head_dim = hidden_size // num_heads
        self.cp_group, self.ep_group = cp_group, ep_group
        self.layer_id = layer_id
        self.moe_combine_chunks, self.moe_dispatch_chunks = moe_combine_chunks, moe_dispatch_chunks
        self.attn_proj_chunks, self.attn_qkv_chunks = attn_proj_chunks, attn_qkv_chunks
        self.activation_func = activation_func
        self.activation = _activation_name(activation_func)
        self.shared_activation = self.activation
        self.capacity_factor = capacity_factor
        self.dropless = capacity_factor is None or capacity_factor <= 0   # keep every routed pair
        self.router_dtype = router_dtype
        self.aux_loss_coeff, self.z_loss_coeff = aux_loss_coeff, z_loss_coeff
        self.init_std = init_std
        self.output_init_std = output_init_std if output_init_std is not None else init_std
        self.norm_type, self.norm_eps = norm_type, norm_eps
        self.comm_mode = comm_mode
        self.fused_ctx = parallel_ctx.fused_ctx if (parallel_ctx is not None and hasattr(parallel_ctx, "fused_ctx")) else None
        self._moe_chunk_config = None
        self.forced_top_idx = None   # [T, k] expert ids replacing the router's selection (see force_routing)

        cp_size, ep_size = comm.group_size(cp_group), comm.group_size(ep_group)
        assert num_experts % ep_size == 0
        nle = num_experts // ep_size
        qpg = num_heads // num_kv_heads
        qkv_size = num_kv_heads * (qpg + 2) * self.head_dim
        fw = 2 * ffn_hidden_size if self.activation == "swiglu" else ffn_hidden_size
        kw = dict(dtype=dtype, device=device)
        self.ln1_weight = nn.Parameter(torch.ones(hidden_size, **kw))
        self.ln2_weight = nn.Parameter(torch.ones(hidden_size, **kw))
        if norm_type == "layernorm":
            self.ln1_bias = nn.Parameter(torch.zeros(hidden_size, **kw))
            self.ln2_bias = nn.Parameter(torch.zeros(hidden_size, **kw))
        else:
            self.ln1_bias = self.ln2_bias = None
        self.qkv_weight = nn.Parameter(torch.empty(qkv_size, hidden_size, **kw))
        self.proj_weight = nn.Parameter(torch.empty(hidden_size, num_heads * self.head_dim, **kw))
        self.router_weight = nn.Parameter(torch.empty(hidden_size, num_experts, **kw))
        self.moe_w1 = nn.Parameter(torch.empty(nle, hidden_size, fw, **kw))
        self.moe_w2 = nn.Parameter(torch.empty(nle, ffn_hidden_size, hidden_size, **kw))
        # Expert weights are reduced over the expert-data-parallel group, not the dense one.
        self.moe_w1.allreduce = False
        self.moe_w2.allreduce = False
        if num_shared_experts > 0:
            sf = (shared_ffn_hidden_size or ffn_hidden_size) * num_shared_experts
            sfw = 2 * sf if self.activation == "swiglu" else sf
            self.shared_w1 = nn.Parameter(torch.empty(hidden_size, sfw, **kw))
            self.shared_w2 = nn.Parameter(torch.empty(sf, hidden_size, **kw))
        else:
            self.shared_w1 = self.shared_w2 = None
        self.attn_overlap_ctx = MultiCardOverlapContext(device, cp_size, cp_size)
        self.moe_overlap_ctx = MultiCardOverlapContext(device, ep_size, ep_size)
        self._rt = LayerRuntime(self)
        self._reset_parameters()

    # ------------------------------------------------------------------ init
    def _reset_parameters(self) -> None:
        """Draw order and layouts follow fluid/layer/transformer.py:981-1056: QKV and router with
        ``init_std``, output projection and FC2 with ``output_init_std``; router drawn as [E, H] and
        expert matrices drawn in the [nle*F, H] / [H, nle*F] layouts, then transposed."""
        with torch.no_grad():
            nn.init.normal_(self.qkv_weight, mean=0.0, std=self.init_std)
            nn.init.normal_(self.proj_weight, mean=0.0, std=self.output_init_std)
            E, H = self.num_experts, self.hidden_size
            tmp = torch.empty(E, H, dtype=self.router_weight.dtype, device=self.router_weight.device)
            nn.init.normal_(tmp, mean=0.0, std=self.init_std)
            self.router_weight.copy_(tmp.t())
            nle, _, fw = self.moe_w1.shape
            tmp1 = torch.empty(nle * fw, H, dtype=self.moe_w1.dtype, device=self.moe_w1.device)
            nn.init.normal_(tmp1, mean=0.0, std=self.init_std)
            self.moe_w1.copy_(tmp1.view(nle, fw, H).transpose(1, 2))
            f = self.moe_w2.shape[1]
            tmp2 = torch.empty(H, nle * f, dtype=self.moe_w2.dtype, device=self.moe_w2.device)
            nn.init.normal_(tmp2, mean=0.0, std=self.output_init_std)
            self.moe_w2.copy_(tmp2.view(H, nle, f).permute(1, 2, 0))
            if self.shared_w1 is not None:
                nn.init.normal_(self.shared_w1, mean=0.0, std=self.init_std)
                nn.init.normal_(self.shared_w2, mean=0.0, std=self.output_init_std)

    # ------------------------------------------------------------------ helpers
    def resolve_mode(self, group_world: int, attention: bool = False, cp_plan=None) -> str:
        if group_world == 1:
            return "a2a"
        fused_ok = self.fused_ctx is not None and (
            not attention or (self.fused_ctx.supports_attention and self.fused_ctx.attention_supported(cp_plan)))
        if self.comm_mode == "auto":
            return "fused" if fused_ok else "p2p"
        if self.comm_mode == "fused":
            if self.fused_ctx is None:
                raise RuntimeError("comm_mode='fused' needs a parallel context with a symmetric heap")
            return "fused" if fused_ok else "p2p"
        return self.comm_mode

    def force_routing(self, top_idx: Optional[torch.Tensor]) -> None:
        """Replace the router's top-k selection by ``top_idx`` (``[tokens, k]`` expert ids) until
        called with None.  Probabilities still come from this layer's logits, so gradients flow as
        usual; used to compare two precisions of the same layer under identical routing."""
        self.forced_top_idx = top_idx

    def set_router_bias(self, bias: Optional[torch.Tensor]) -> None:
        """A fixed (not trained) prior ``[num_experts]`` added to the router logits before the top-k
        selection, e.g. a Zipf prior that makes the expert load skewed."""
        self.router_logit_bias = None if bias is None else bias.detach().to(
            device=self.router_weight.device, dtype=torch.float32)

    def attach_fused(self, fused_ctx) -> None:
        self.fused_ctx = fused_ctx
        self._rt.sig = None

    def forward(self, x: torch.Tensor, rotary_pos_emb: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: ``[seq_local, batch, hidden]``; rotary_pos_emb: ``[seq_full, 1, 1, rot_dim]`` or None."""
        self._rt.grad_enabled = torch.is_grad_enabled()
        return TransformerLayerFunction.apply(
            x, self.ln1_weight, self.ln1_bias, self.ln2_weight, self.ln2_bias, self.qkv_weight,
            self.proj_weight, self.router_weight, self.moe_w1, self.moe_w2, self.shared_w1,
            self.shared_w2, rotary_pos_emb, self._rt)


class TransformerModel(nn.Module):
    """A stack of blocks (fluid/layer/transformer.py:1152-1294)."""

    def __init__(self, num_layers: int, hidden_size: int, num_heads: int, num_kv_heads: int,
                 ffn_hidden_size: int, num_experts: int, top_k: int, cp_group=None, ep_group=None,
                 moe_combine_chunks: int = 1, moe_dispatch_chunks: int = 1, attn_proj_chunks: int = 1,
                 attn_qkv_chunks: int = 1, activation_func=None, capacity_factor: float = 1.0,
                 init_std: float = 0.02, dtype: torch.dtype = torch.bfloat16, device=None,
                 router_dtype: torch.dtype = torch.bfloat16, aux_loss_coeff: float = 0.0,
                 z_loss_coeff: float = 0.0, **layer_kwargs):
        super().__init__()
        self.num_layers = num_layers
        out_std = init_std / math.sqrt(2.0 * num_layers)
        self.layers = nn.ModuleList([
            TransformerLayer(hidden_size, num_heads, num_kv_heads, ffn_hidden_size, num_experts, top_k,
                             cp_group, ep_group, i, moe_combine_chunks, moe_dispatch_chunks,
                             attn_proj_chunks, attn_qkv_chunks, activation_func, capacity_factor,
                             init_std, out_std, dtype, device, router_dtype, aux_loss_coeff,
                             z_loss_coeff, **layer_kwargs)
            for i in range(num_layers)])

    def forward(self, x: torch.Tensor, rotary_pos_emb: Optional[torch.Tensor] = None) -> torch.Tensor:
        for layer in self.layers:
            x = layer(x, rotary_pos_emb)
        return x

    def prepare_chunk_status(self, x: torch.Tensor) -> dict:
        """Report, for the given input shape, the chunk count each backward region will use
        (requests that do not divide the work fall back to fewer chunks)."""
        s_loc, b, _ = x.shape
        L = self.layers[0]
        ep = comm.group_size(L.ep_group)
        nle = L.num_experts // ep
        cap = router_ops.expert_capacity(s_loc * b, L.top_k, L.num_experts, L.capacity_factor)
        cfg = moe_mod.build_moe_chunk_config(L.moe_combine_chunks, L.moe_dispatch_chunks, nle, cap)
        status = {
            "moe_combine": cfg["moe_combine"].num_chunks, "moe_dispatch": cfg["moe_dispatch"].num_chunks,
            "attn_proj": L.attn_proj_chunks if s_loc % max(1, L.attn_proj_chunks) == 0 else 1,
            "attn_qkv": L.attn_qkv_chunks if s_loc % max(1, L.attn_qkv_chunks) == 0 else 1,
        }
        requested = {"moe_combine": L.moe_combine_chunks, "moe_dispatch": L.moe_dispatch_chunks,
                     "attn_proj": L.attn_proj_chunks, "attn_qkv": L.attn_qkv_chunks}
        for k_, v_ in status.items():
            if v_ != requested[k_]:
                moe_mod._warn_once(f"status:{k_}", f"region {k_}: requested {requested[k_]} chunks, using {v_}")
        return status

    def expert_params(self):
        return [p for l in self.layers for p in (l.moe_w1, l.moe_w2)]

    def shared_params(self):
        ex = {id(p) for p in self.expert_params()}
        return [p for p in self.parameters() if id(p) not in ex]

    def setup_ar_buffer(self, accumulate_in_fp32: bool = True, allocator=None) -> None:
        """Register parameters in the scheduler's flat gradient buffers in backward order (last
        layer first), dense and expert parameters separately
        (fluid/layer/transformer.py:1263-1288)."""
        sched = get_backward_scheduler()
        shared, expert = [], []
        for layer in reversed(self.layers):
            expert += [layer.moe_w2, layer.moe_w1]
            shared += [p for p in (layer.router_weight, layer.shared_w2, layer.shared_w1, layer.ln2_weight,
                                   layer.ln2_bias, layer.proj_weight, layer.qkv_weight, layer.ln1_weight,
                                   layer.ln1_bias) if p is not None]
        sched.setup_ar_buffer(shared, accumulate_in_fp32, allocator)
        sched.setup_expert_ar_buffer(expert, accumulate_in_fp32, allocator)
