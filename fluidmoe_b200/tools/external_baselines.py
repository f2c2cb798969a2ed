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


def megatron_config_kwargs(cfg: dict, dtype=torch.bfloat16, cp_size: int = 1, ep_size: int = 1) -> dict:
    """Keyword arguments of Megatron-Core's ``TransformerConfig`` for a preset of
    ``tools.model_configs`` (keys ``hidden_size, num_heads, num_kv_heads, ffn_hidden, num_experts,
    top_k, num_layers, capacity_factor, activation, norm_type``): all-to-all dispatcher with padded
    capacity and grouped GEMM, all-to-all context parallelism, TP = PP = 1
    (tools/megatron_baseline.py:118-160 of the reference)."""
    return dict(
        num_layers=int(cfg["num_layers"]), hidden_size=int(cfg["hidden_size"]),
        num_attention_heads=int(cfg["num_heads"]), num_query_groups=int(cfg["num_kv_heads"]),
        ffn_hidden_size=int(cfg["ffn_hidden"]), num_moe_experts=int(cfg["num_experts"]),
        moe_router_topk=int(cfg["top_k"]), moe_grouped_gemm=True, moe_token_dispatcher_type="alltoall",
        moe_expert_capacity_factor=float(cfg.get("capacity_factor", 1.0)),
        moe_pad_expert_input_to_capacity=True, add_bias_linear=False, bf16=dtype == torch.bfloat16,
        params_dtype=dtype, cp_comm_type="a2a", attention_dropout=0.0, hidden_dropout=0.0,
        tensor_model_parallel_size=1, pipeline_model_parallel_size=1, context_parallel_size=int(cp_size),
        expert_model_parallel_size=int(ep_size),
        gated_linear_unit=cfg.get("activation", "gelu") == "swiglu",
        normalization="RMSNorm" if cfg.get("norm_type", "layernorm") == "rmsnorm" else "LayerNorm")


def build_megatron_baseline(cfg: dict, cp_group=None, ep_group=None, dtype=torch.bfloat16, device="cuda"):
    """A stack of Megatron-Core MoE transformer layers with the preset's shapes."""
    _need("megatron.core", "transformer_engine")
    from megatron.core.models.gpt.gpt_layer_specs import get_gpt_layer_with_transformer_engine_spec
    from megatron.core.transformer.transformer_block import TransformerBlock
    from megatron.core.transformer.transformer_config import TransformerConfig
    import torch.distributed as dist

    size = lambda g: dist.get_world_size(g) if (g is not None and dist.is_initialized()) else 1  # noqa: E731
    tc = TransformerConfig(**megatron_config_kwargs(cfg, dtype, size(cp_group), size(ep_group)))
    spec = get_gpt_layer_with_transformer_engine_spec(num_experts=int(cfg["num_experts"]), moe_grouped_gemm=True)
    return TransformerBlock(tc, spec, post_layer_norm=False).to(device)


def deepspeed_block_kwargs(cfg: dict, ep_size: int = 1) -> dict:
    """Shapes of the DeepSpeed arm for a preset: Ulysses attention over all heads (the wrapper has no
    grouped-query form, so K and V get ``num_heads`` heads), ``deepspeed.moe.layer.MoE`` with GELU
    experts, token dropping at the preset's capacity factor
    (tools/deepspeed_ulysses_baseline.py:49-279 of the reference)."""
    return dict(hidden=int(cfg["hidden_size"]), heads=int(cfg["num_heads"]), ffn=int(cfg["ffn_hidden"]),
                num_experts=int(cfg["num_experts"]), ep_size=int(ep_size), k=int(cfg["top_k"]),
                capacity_factor=float(cfg.get("capacity_factor", 1.0)), num_layers=int(cfg["num_layers"]))


def build_deepspeed_ulysses_baseline(cfg: dict, sp_group=None, ep_size: int = 1, dtype=torch.bfloat16,
                                     device="cuda"):
    """A stack of blocks made of DeepSpeed's Ulysses attention wrapper and its MoE layer."""
    _need("deepspeed")
    import deepspeed
    from deepspeed.moe.layer import MoE
    from deepspeed.sequence.layer import DistributedAttention

    kw = deepspeed_block_kwargs(cfg, ep_size)
    H, nh = kw["hidden"], kw["heads"]
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
            expert = torch.nn.Sequential(torch.nn.Linear(H, kw["ffn"], bias=False), torch.nn.GELU(),
                                         torch.nn.Linear(kw["ffn"], H, bias=False))
            self.moe = MoE(H, expert, num_experts=kw["num_experts"], ep_size=kw["ep_size"], k=kw["k"],
                           capacity_factor=kw["capacity_factor"], drop_tokens=True)

        def forward(self, x):                        # [s_local, b, H]
            s, b, _ = x.shape
            q, k, v = self.qkv(self.ln1(x)).view(s, b, 3, nh, hd).unbind(2)
            x = x + self.proj(self.attn(q, k, v).reshape(s, b, H))
            y, _, _ = self.moe(self.ln2(x))
            return x + y

    del deepspeed
    return torch.nn.Sequential(*[_Block() for _ in range(kw["num_layers"])]).to(device=device, dtype=dtype)
