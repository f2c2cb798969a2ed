"""A complete sequence-parallel MoE language model around the transformer blocks:
token embedding -> N blocks -> final norm -> LM head -> cross-entropy on shifted ids.

Every rank holds a contiguous block of the sequence; embedding, head and loss are local to the
rank's positions, the blocks exchange data over the sequence-/expert-parallel group.  Weight
gradients of the head go through the backward scheduler like those of the blocks, so the final
norm and head gradients are the first entries of the dense flat buffer and can be reduced in the
earliest communication gaps (fluid/setup.py:104-140 does this with autograd hooks under Megatron).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native
from ..ops import gemm, norm
from ..ops.rope import make_rope_freqs
from ..parallel import comm
from ..parallel.scheduler import get_backward_scheduler
from .attention import _register_dense_dw
from .transformer import TransformerModel


class _FinalNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps, kind):
        y, mean, rstd = norm.norm_fwd(x, w, b, eps, kind)
        ctx.kind, ctx.params = kind, (w, b)
        ctx.save_for_backward(x, mean if mean is not None else rstd, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, mean, rstd = ctx.saved_tensors
        w, b = ctx.params
        ln = ctx.kind == "layernorm"
        dx, dw, db = norm.norm_bwd(dy.contiguous(), x, w, mean if ln else None, rstd, ctx.kind, b is not None)
        sched = get_backward_scheduler()
        sched.register_dw_task("final_norm.w", -1, lambda: dw, w)
        if b is not None:
            sched.register_dw_task("final_norm.b", -1, lambda: db, b)
        return dx, None, None, None, None


class _Embedding(torch.autograd.Function):
    """Token embedding whose backward adds the touched rows straight into the parameter's fp32
    gradient buffer (``weight.main_grad``, set by ``FluidDDP``): a step touches ``tokens`` of the
    ``vocab`` rows, so this moves ``tokens x H`` values instead of building a dense ``[vocab, H]``
    gradient, converting it and adding it over the whole table.  Without a gradient buffer it
    returns the dense gradient like ``F.embedding``.  Rows that occur several times are summed with
    floating-point atomics on the GPU, i.e. in no fixed order."""

    @staticmethod
    def forward(ctx, ids, weight):
        ctx.save_for_backward(ids)
        ctx.weight = weight
        return F.embedding(ids, weight)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.weight
        flat_ids, flat_dy = ids.reshape(-1), dy.reshape(-1, dy.shape[-1])
        main = getattr(w, "main_grad", None)
        if main is not None and main.dtype == torch.float32:
            main.index_add_(0, flat_ids, flat_dy.float())
            return None, None
        grad = torch.zeros_like(w, dtype=torch.float32).index_add_(0, flat_ids, flat_dy.float())
        return None, grad.to(w.dtype)


class _HeadLoss(torch.autograd.Function):
    """LM head GEMM + mean cross-entropy; the backward produces dh and queues the head dW."""

    @staticmethod
    def forward(ctx, h, w, labels):
        logits = gemm.gemm_nt(h, w)                          # [T, V]
        if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.shape[1] % 8 == 0 \
                and _native.available():
            # fused path: the kernel leaves d(loss)/d(logits) for a mean loss in `logits`
            from ..ops import elementwise
            n = (labels >= 0).sum().clamp(min=1)
            rows = elementwise.cross_entropy_(logits, labels, 1.0)
            loss = rows.sum() / n
            ctx.save_for_backward(h, logits, n)
            ctx.w, ctx.fused = w, True
            return loss
        ctx.fused = False
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1)
        valid = labels >= 0
        tgt = lf.gather(1, labels.clamp(min=0).unsqueeze(1)).squeeze(1)
        n = valid.sum().clamp(min=1)
        loss = ((lse - tgt) * valid).sum() / n
        ctx.save_for_backward(h, logits, lse, labels, n)
        ctx.w = w
        return loss

    @staticmethod
    def backward(ctx, dloss):
        w = ctx.w
        if ctx.fused:
            h, dlogits, n = ctx.saved_tensors
            # d(loss)/d(logits) as the kernel left it is for a sum; the factor dloss / n goes onto the
            # two [T, H] tensors around it instead of one pass over the [T, V] logits
            scale = (dloss / n).float()
            dh = gemm.gemm_nn(dlogits, w).mul_(scale)
            _register_dense_dw("lm_head", -1, h * scale, dlogits, w)
            return dh, None, None
        h, logits, lse, labels, n = ctx.saved_tensors
        p = torch.exp(logits.float() - lse.unsqueeze(1))
        valid = (labels >= 0).unsqueeze(1)
        p.scatter_add_(1, labels.clamp(min=0).unsqueeze(1), -torch.ones_like(lse).unsqueeze(1))
        dlogits = (p * valid * (dloss / n)).to(h.dtype)
        dh = gemm.gemm_nn(dlogits, w)
        _register_dense_dw("lm_head", -1, h, dlogits, w)
        return dh, None, None


class MoEGPT(nn.Module):
    def __init__(self, vocab_size: int, num_layers: int, hidden_size: int, num_heads: int,
                 num_kv_heads: int, ffn_hidden_size: int, num_experts: int, top_k: int, cp_group=None,
                 ep_group=None, dtype=torch.bfloat16, device=None, rope_base: float = 10000.0,
                 rot_dim: Optional[int] = None, init_std: float = 0.02, **layer_kwargs):
        super().__init__()
        self.cp_group = cp_group
        self.hidden_size = hidden_size
        self.head_dim = hidden_size // num_heads
        self.rot_dim = rot_dim if rot_dim is not None else self.head_dim
        self.rope_base = rope_base
        self.norm_type = layer_kwargs.get("norm_type", "layernorm")
        self.norm_eps = layer_kwargs.get("norm_eps", 1e-5)
        self.embedding = nn.Embedding(vocab_size, hidden_size, dtype=dtype, device=device)
        nn.init.normal_(self.embedding.weight, std=init_std)
        self.decoder = TransformerModel(num_layers, hidden_size, num_heads, num_kv_heads, ffn_hidden_size,
                                        num_experts, top_k, cp_group, ep_group, dtype=dtype, device=device,
                                        init_std=init_std, **layer_kwargs)
        self.final_norm_weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.final_norm_bias = (nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=device))
                                if self.norm_type == "layernorm" else None)
        self.lm_head = nn.Parameter(torch.empty(vocab_size, hidden_size, dtype=dtype, device=device))
        nn.init.normal_(self.lm_head, std=init_std)
        self._freqs = None

    def rotary(self, seq_full: int, device) -> torch.Tensor:
        if self._freqs is None or self._freqs.shape[0] != seq_full or self._freqs.device != device:
            self._freqs = make_rope_freqs(seq_full, self.rot_dim, self.rope_base, device)
        return self._freqs

    def forward(self, ids: torch.Tensor, labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        """ids: ``[seq_local, batch]`` token ids of this rank's block; labels: same shape (next-token
        targets, negative = ignore).  Returns the mean loss over this rank's positions, or the
        final hidden states when ``labels`` is None."""
        s_loc, b = ids.shape
        P = comm.group_size(self.cp_group)
        x = _Embedding.apply(ids, self.embedding.weight)          # [s_loc, b, H]
        x = self.decoder(x, self.rotary(s_loc * P, ids.device))
        h = _FinalNorm.apply(x.reshape(s_loc * b, -1), self.final_norm_weight, self.final_norm_bias,
                             self.norm_eps, self.norm_type)
        if labels is None:
            return h.view(s_loc, b, -1)
        return _HeadLoss.apply(h, self.lm_head, labels.reshape(-1))

    def setup_ar_buffer(self, accumulate_in_fp32: bool = True, allocator=None) -> None:
        """Flat gradient buffers in backward order: head and final norm first, then the blocks from
        last to first, then the embedding; expert weights in their own buffer."""
        sched = get_backward_scheduler()
        shared = [self.lm_head, self.final_norm_weight]
        if self.final_norm_bias is not None:
            shared.append(self.final_norm_bias)
        expert = []
        for layer in reversed(self.decoder.layers):
            expert += [layer.moe_w2, layer.moe_w1]
            shared += [p for p in (layer.router_weight, layer.shared_w2, layer.shared_w1, layer.ln2_weight,
                                   layer.ln2_bias, layer.proj_weight, layer.qkv_weight, layer.ln1_weight,
                                   layer.ln1_bias) if p is not None]
        sched.setup_ar_buffer(shared, accumulate_in_fp32, allocator)
        sched.setup_expert_ar_buffer(expert, accumulate_in_fp32, allocator)
