"""Baselines built from other frameworks, for side-by-side block benchmarks.

The reference compares itself with a Megatron-Core block (Transformer Engine layer spec, all-to-all
token dispatcher, padded capacity, grouped GEMM, context-parallel attention with ``cp_comm_type =
"a2a"``; tools/megatron_baseline.py:60-171) and with a DeepSpeed block (Ulysses
``DistributedAttention`` plus ``deepspeed.moe.layer.MoE``; tools/deepspeed_ulysses_baseline.py:49-279).
Neither package is a dependency of this framework.  The builders below assemble the same two blocks
when the packages are importable and raise ``BaselineUnavailable`` (with the missing package named)
when they are not; ``available()`` reports which arms can run.  The built-in baseline that needs no
other package is this framework's own ``fluidmoe-f`` arm (scheduler off, library all-to-all).
"""
from __future__ import annotations

import importlib
from typing import Dict

import torch


class BaselineUnavailable(RuntimeError):
    pass


def _need(*modules: str):
    out = []
    for m in modules:
        try:
            out.append(importlib.import_module(m))
        except Exception as e:  # noqa: BLE001 - any import failure means the arm cannot run
            raise BaselineUnavailable(f"baseline needs the '{m.split('.')[0]}' package: {e}") from e
    return out


def available() -> Dict[str, bool]:
    res = {}
    for name, mods in (("megatron", ("megatron.core", "transformer_engine")), ("deepspeed", ("deepspeed",))):
        try:
            _need(*mods)
            res[name] = True
        except BaselineUnavailable:
            res[name] = False
    return res


def build_megatron_baseline(cfg: dict, cp_group=None, ep_group=None, dtype=torch.bfloat16, device="cuda"):
    """A stack of Megatron-Core MoE transformer layers with the preset's shapes.  ``cfg`` is a preset
    of ``tools.model_configs`` (hidden_size, num_heads, num_kv_heads, ffn_hidden_size, num_experts,
    top_k, num_layers, capacity_factor)."""
    _need("megatron.core", "transformer_engine")
    from megatron.core.models.gpt.gpt_layer_specs import get_gpt_layer_with_transformer_engine_spec
    from megatron.core.transformer.transformer_block import TransformerBlock
    from megatron.core.transformer.transformer_config import TransformerConfig

    tc = TransformerConfig(
        num_layers=cfg["num_layers"], hidden_size=cfg["hidden_size"], num_attention_heads=cfg["num_heads"],
        num_query_groups=cfg["num_kv_heads"], ffn_hidden_size=cfg["ffn_hidden_size"],
        num_moe_experts=cfg["num_experts"], moe_router_topk=cfg["top_k"], moe_grouped_gemm=True,
        moe_token_dispatcher_type="alltoall", moe_expert_capacity_factor=cfg.get("capacity_factor", 1.0),
        moe_pad_expert_input_to_capacity=True, add_bias_linear=False, bf16=dtype == torch.bfloat16,
        params_dtype=dtype, cp_comm_type="a2a", attention_dropout=0.0, hidden_dropout=0.0,
        gated_linear_unit=cfg.get("activation", "gelu") == "swiglu",
        normalization="RMSNorm" if cfg.get("norm", "layernorm") == "rmsnorm" else "LayerNorm")
    spec = get_gpt_layer_with_transformer_engine_spec(num_experts=cfg["num_experts"], moe_grouped_gemm=True)
    return TransformerBlock(tc, spec, post_layer_norm=False).to(device)


def build_deepspeed_ulysses_baseline(cfg: dict, sp_group=None, ep_size: int = 1, dtype=torch.bfloat16,
                                     device="cuda"):
    """A stack of blocks made of DeepSpeed's Ulysses attention wrapper and its MoE layer."""
    _need("deepspeed")
    import deepspeed
    from deepspeed.moe.layer import MoE
    from deepspeed.sequence.layer import DistributedAttention

    H, nh = cfg["hidden_size"], cfg["num_heads"]
    hd = H // nh

    class _LocalAttention(torch.nn.Module):
        def forward(self, q, k, v, *a, **kw):       # [s, b, h, d] after the Ulysses exchange
            o = torch.nn.functional.scaled_dot_product_attention(
                q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3), is_causal=True)
            return o.permute(2, 0, 1, 3)

    class _Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = torch.nn.LayerNorm(H), torch.nn.LayerNorm(H)
            self.qkv, self.proj = torch.nn.Linear(H, 3 * H, bias=False), torch.nn.Linear(H, H, bias=False)
            self.attn = DistributedAttention(_LocalAttention(), sp_group, scatter_idx=2, gather_idx=0)
            expert = torch.nn.Sequential(torch.nn.Linear(H, cfg["ffn_hidden_size"], bias=False), torch.nn.GELU(),
                                         torch.nn.Linear(cfg["ffn_hidden_size"], H, bias=False))
            self.moe = MoE(H, expert, num_experts=cfg["num_experts"], ep_size=ep_size, k=cfg["top_k"],
                           capacity_factor=cfg.get("capacity_factor", 1.0), drop_tokens=True)

        def forward(self, x):                        # [s_local, b, H]
            s, b, _ = x.shape
            q, k, v = self.qkv(self.ln1(x)).view(s, b, 3, nh, hd).unbind(2)
            x = x + self.proj(self.attn(q, k, v).reshape(s, b, H))
            y, _, _ = self.moe(self.ln2(x))
            return x + y

    del deepspeed
    return torch.nn.Sequential(*[_Block() for _ in range(cfg["num_layers"])]).to(device=device, dtype=dtype)
