"""A second, independent statement of one MoE transformer block, written with plain torch
operators only and differentiated by autograd.

It shares no code with ``fluidmoe_b200.models``: normalisation, projections, rotate-half RoPE,
causal grouped-query attention in fp32, the top-k-then-softmax router with per-expert capacity
dropping, dense per-expert MLPs weighted by the routing probability, shared experts, and the two
router regularisers.  The hand-written backward of the library's block
(fluid/layer/transformer.py:396-810 is its counterpart in the reference) is verified against the
gradients autograd derives from this module.

Routing and capacity are decided per rank (every rank routes its own ``seq_local * batch`` tokens),
attention sees the whole sequence: ``world`` tells the oracle how the sequence would be split.
"""
import math

import torch
import torch.nn.functional as F


def _norm(x, w, b, kind, eps):
    if kind == "layernorm":
        return F.layer_norm(x, (x.shape[-1],), w, b, eps)
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(t, angles):
    """t ``[s, b, h, d]``, angles ``[s, 1, 1, rot]`` (two equal halves): t*cos + rotate_half(t)*sin."""
    rot = angles.shape[-1]
    tr, rest = t[..., :rot], t[..., rot:]
    x1, x2 = tr[..., : rot // 2], tr[..., rot // 2:]
    out = tr * torch.cos(angles) + torch.cat((-x2, x1), dim=-1) * torch.sin(angles)
    return torch.cat((out, rest), dim=-1)


def _act(pre, kind):
    if kind == "swiglu":
        gate, up = pre.chunk(2, dim=-1)
        return F.silu(gate) * up
    if kind == "silu":
        return F.silu(pre)
    return F.gelu(pre)          # exact (erf) form


def block_forward(x, P, *, num_heads, num_kv_heads, top_k, world, activation="gelu", norm_type="layernorm",
                  eps=1e-5, capacity_factor=1.0, rotary=None, aux_loss_coeff=0.0, z_loss_coeff=0.0):
    """x ``[s_full, b, H]``; ``P`` maps the layer's state-dict names to FULL tensors (all experts:
    ``moe_w1 [E, H, F or 2F]``, ``moe_w2 [E, F, H]``).  Returns ``(y, regulariser)`` where the
    regulariser is the sum over ranks of the load-balancing and z losses whose gradients the
    library injects analytically."""
    S, b, H = x.shape
    d = H // num_heads
    qpg = num_heads // num_kv_heads
    E = P["router_weight"].shape[1]
    # ---- attention half ----
    h = _norm(x, P["ln1_weight"], P.get("ln1_bias"), norm_type, eps)
    qkv = (h @ P["qkv_weight"].t()).view(S, b, num_kv_heads, qpg + 2, d)
    q = qkv[:, :, :, :qpg].reshape(S, b, num_heads, d)
    k, v = qkv[:, :, :, qpg], qkv[:, :, :, qpg + 1]
    if rotary is not None:
        q, k = _rope(q, rotary), _rope(k, rotary)
    kq = k.repeat_interleave(qpg, dim=2)
    vq = v.repeat_interleave(qpg, dim=2)
    sc = torch.einsum("sbhd,tbhd->bhst", q, kq) / math.sqrt(d)
    mask = torch.ones(S, S, dtype=torch.bool).tril()
    sc = sc.masked_fill(~mask, float("-inf"))
    attn = torch.einsum("bhst,tbhd->sbhd", torch.softmax(sc, dim=-1), vq).reshape(S, b, H)
    h1 = x + attn @ P["proj_weight"].t()
    # ---- MoE half, routed rank by rank ----
    ln2 = _norm(h1, P["ln2_weight"], P.get("ln2_bias"), norm_type, eps)
    s_loc = S // world
    T = s_loc * b
    dropless = capacity_factor is None or capacity_factor <= 0
    cap = T if dropless else int(math.ceil(T * top_k / E * capacity_factor))
    outs, routed, sel_probs, sel_idx, reg = [], [], [], [], x.new_zeros(())
    for r in range(world):
        tok = ln2[r * s_loc:(r + 1) * s_loc].reshape(T, H)
        logits = tok.float() @ P["router_weight"].float()
        top_logits, top_idx = torch.topk(logits, top_k, dim=-1)
        top_probs = torch.softmax(top_logits, dim=-1)
        probs = torch.zeros(T, E).scatter(1, top_idx, top_probs)
        rmap = torch.zeros(T, E, dtype=torch.bool).scatter(1, top_idx, True)
        if cap < T:
            keep = torch.topk(probs.detach(), cap, dim=0).indices
            rmap = rmap & torch.zeros(T, E, dtype=torch.bool).scatter(0, keep, True)
            probs = probs * rmap
        out = torch.zeros(T, H)
        for e in range(E):
            rows = rmap[:, e].nonzero().squeeze(1)
            if rows.numel():
                a = _act(tok[rows] @ P["moe_w1"][e], activation) * probs[rows, e].unsqueeze(1).to(tok.dtype)
                out = out.index_add(0, rows, a @ P["moe_w2"][e])
        if P.get("shared_w1") is not None:
            out = out + _act(tok @ P["shared_w1"], activation) @ P["shared_w2"]
        outs.append(out.view(s_loc, b, H))
        routed.append(rmap.sum(0).float())
        sel_probs.append(top_probs)
        sel_idx.append(top_idx)
        if z_loss_coeff > 0.0:
            reg = reg + z_loss_coeff / T * torch.logsumexp(logits, dim=-1).pow(2).sum()
    if aux_loss_coeff > 0.0:
        tpe = torch.stack(routed).sum(0)                  # tokens per expert over the whole group
        coef = E * aux_loss_coeff / (top_k * float(T * world) ** 2)
        for top_probs, top_idx in zip(sel_probs, sel_idx):
            reg = reg + coef * (tpe[top_idx] * top_probs).sum()
    return h1 + torch.cat(outs, dim=0), reg


def full_params_from_layers(layers):
    """Full (all experts) fp32 leaf tensors from one layer per expert-parallel rank."""
    first = layers[0]
    P = {}
    for name, p in first.named_parameters():
        if name in ("moe_w1", "moe_w2"):
            t = torch.cat([dict(l.named_parameters())[name].detach() for l in layers], dim=0)
        else:
            t = p.detach()
        P[name] = t.clone().float().requires_grad_(True)
    return P
