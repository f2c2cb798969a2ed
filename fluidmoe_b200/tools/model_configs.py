"""Model presets.  The first six reproduce the shapes of the reference's presets
(tools/model_configs.py:32-163); the others are the configurations named by the build's
benchmark plan (SwiGLU Mixtral layer, fine-grained MoE with shared experts)."""
from __future__ import annotations

from typing import Dict, List

MODEL_CONFIGS: Dict[str, dict] = {
    "mixtral_8x7b": dict(hidden_size=4096, num_heads=32, num_kv_heads=8, ffn_hidden=14336, num_experts=8,
                         top_k=2, num_layers=2, seq_len=4096, batch_size=2, capacity_factor=1.0),
    "dbrx": dict(hidden_size=6144, num_heads=48, num_kv_heads=8, ffn_hidden=10752, num_experts=16, top_k=4,
                 num_layers=6, seq_len=8192, batch_size=1, capacity_factor=1.0),
    "phi_3_5_moe": dict(hidden_size=4096, num_heads=32, num_kv_heads=8, ffn_hidden=6400, num_experts=16,
                        top_k=2, num_layers=8, seq_len=8192, batch_size=1, capacity_factor=1.0),
    "olmoe_1b_7b": dict(hidden_size=2048, num_heads=16, num_kv_heads=16, ffn_hidden=1024, num_experts=64,
                        top_k=8, num_layers=4, seq_len=4096, batch_size=2, capacity_factor=1.0),
    "deepseek_v3_mha_proxy": dict(hidden_size=7168, num_heads=128, num_kv_heads=128, ffn_hidden=2048,
                                  num_experts=256, top_k=8, num_layers=2, seq_len=4096, batch_size=1,
                                  capacity_factor=1.0),
    "glm4_5_air_mha_proxy": dict(hidden_size=4096, num_heads=32, num_kv_heads=8, ffn_hidden=1408,
                                 num_experts=128, top_k=8, num_layers=4, seq_len=4096, batch_size=1,
                                 capacity_factor=1.0),
    # configurations of the benchmark plan
    "mixtral_8x7b_swiglu": dict(hidden_size=4096, num_heads=32, num_kv_heads=8, ffn_hidden=14336,
                                num_experts=8, top_k=2, num_layers=4, seq_len=4096, batch_size=1,
                                capacity_factor=1.0, activation="swiglu", norm_type="rmsnorm", vocab_size=32000),
    "fine_grained_64e": dict(hidden_size=2048, num_heads=16, num_kv_heads=16, ffn_hidden=1408, num_experts=64,
                             top_k=6, num_layers=1, seq_len=8192, batch_size=1, capacity_factor=1.0,
                             activation="swiglu", norm_type="rmsnorm", num_shared_experts=2),
    # block benchmarks of the plan: the MoE half and the attention half of the flagship block on their
    # own, the whole block, and the fine-grained MoE layer with a skewed (Zipf) expert load.
    # ``seq_per_rank`` keeps the work per rank fixed as the group grows (weak scaling).
    "cfg2_mixtral_moe_layer": dict(hidden_size=4096, num_heads=32, num_kv_heads=8, ffn_hidden=14336, num_experts=8,
                                   top_k=2, num_layers=1, seq_len=4096, seq_per_rank=4096, batch_size=1,
                                   capacity_factor=1.0, activation="swiglu", norm_type="rmsnorm",
                                   has_attention=False),
    "cfg3_ulysses_attention_block": dict(hidden_size=4096, num_heads=32, num_kv_heads=8, ffn_hidden=14336,
                                         num_experts=8, top_k=2, num_layers=1, seq_len=4096, seq_per_rank=4096,
                                         batch_size=1, capacity_factor=1.0, activation="swiglu",
                                         norm_type="rmsnorm", has_moe=False, rope=True),
    "cfg23_mixtral_block": dict(hidden_size=4096, num_heads=32, num_kv_heads=8, ffn_hidden=14336, num_experts=8,
                                top_k=2, num_layers=1, seq_len=4096, seq_per_rank=4096, batch_size=1,
                                capacity_factor=1.0, activation="swiglu", norm_type="rmsnorm", rope=True),
    "cfg5_fine_grained_moe_layer": dict(hidden_size=2048, num_heads=16, num_kv_heads=16, ffn_hidden=1408,
                                        num_experts=64, top_k=6, num_layers=1, seq_len=8192, seq_per_rank=8192,
                                        batch_size=1, capacity_factor=0.0, activation="swiglu", norm_type="rmsnorm",
                                        num_shared_experts=2, has_attention=False, zipf_s=1.1),
    "cfg5_fine_grained_block": dict(hidden_size=2048, num_heads=16, num_kv_heads=16, ffn_hidden=1408,
                                    num_experts=64, top_k=6, num_layers=1, seq_len=8192, seq_per_rank=8192,
                                    batch_size=1, capacity_factor=0.0, activation="swiglu", norm_type="rmsnorm",
                                    num_shared_experts=2, zipf_s=1.1, rope=True),
    "tiny_test": dict(hidden_size=256, num_heads=8, num_kv_heads=4, ffn_hidden=512, num_experts=4, top_k=2,
                      num_layers=1, seq_len=128, batch_size=2, capacity_factor=1.0),
}


def get_model_config(name: str) -> dict:
    if name not in MODEL_CONFIGS:
        raise KeyError(f"unknown model preset {name!r}; known: {', '.join(list_model_names())}")
    return dict(MODEL_CONFIGS[name])


def reference_variant(cfg: dict) -> dict:
    """The nearest configuration the reference implementation can express: non-gated GELU experts
    (FFN widened by 3/2 when the preset is SwiGLU, which keeps FLOPs and weight bytes), LayerNorm,
    padded capacity 1.0 (it has no dropless routing), no shared experts, always both halves of the
    block, no router prior."""
    out = dict(cfg)
    if out.get("activation", "gelu") == "swiglu":
        out["ffn_hidden"] = int(out["ffn_hidden"]) * 3 // 2
    out.update(activation="gelu", norm_type="layernorm", num_shared_experts=0, has_attention=True, has_moe=True,
               zipf_s=0.0)
    if float(out.get("capacity_factor", 1.0)) <= 0.0:
        out["capacity_factor"] = 1.0
    return out


def list_model_names() -> List[str]:
    return sorted(MODEL_CONFIGS)
