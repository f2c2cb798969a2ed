"""Adapter that plugs the block into a Megatron-Core GPT model (import-guarded).

``FluidTransformerLayer`` maps a Megatron ``TransformerConfig`` onto :class:`TransformerLayer`;
``get_fluid_gpt_layer_spec()`` (alias ``get_fluid_custom_layers()``, the name used by the
reference's README:81,91) returns the ``ModuleSpec``.  Chunk counts come from the environment
variables ``FLUIDMOE_{MOE_COMBINE,MOE_DISPATCH,ATTN_PROJ,ATTN_QKV}_CHUNKS`` as in
fluid/layer/fluid_spec.py:26-130.  Without megatron-core the functions raise ImportError with a
clear message; everything else in this package works without Megatron.
"""
from __future__ import annotations

import os

import torch

from .transformer import TransformerLayer


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def layer_kwargs_from_config(config, layer_number: int = 1) -> dict:
    """Translate the fields of a Megatron ``TransformerConfig`` (or any object with the same
    attribute names) into :class:`TransformerLayer` keyword arguments."""
    act = getattr(config, "activation_func", None)
    gated = bool(getattr(config, "gated_linear_unit", False))
    act_name = getattr(act, "__name__", "gelu") if act is not None else "gelu"
    if gated and "silu" in act_name:
        act_name = "swiglu"
    cf = getattr(config, "moe_expert_capacity_factor", None)
    return dict(
        hidden_size=config.hidden_size, num_heads=config.num_attention_heads,
        num_kv_heads=getattr(config, "num_query_groups", None) or config.num_attention_heads,
        ffn_hidden_size=getattr(config, "moe_ffn_hidden_size", None) or config.ffn_hidden_size,
        num_experts=config.num_moe_experts, top_k=config.moe_router_topk,
        layer_id=layer_number - 1,
        moe_combine_chunks=_env_int("FLUIDMOE_MOE_COMBINE_CHUNKS", 1),
        moe_dispatch_chunks=_env_int("FLUIDMOE_MOE_DISPATCH_CHUNKS", 1),
        attn_proj_chunks=_env_int("FLUIDMOE_ATTN_PROJ_CHUNKS", 1),
        attn_qkv_chunks=_env_int("FLUIDMOE_ATTN_QKV_CHUNKS", 1),
        activation_func=act_name, capacity_factor=cf if cf is not None else 1.0,
        init_std=getattr(config, "init_method_std", 0.02),
        output_init_std=getattr(config, "init_method_std", 0.02) / (2.0 * max(1, getattr(config, "num_layers", 1))) ** 0.5,
        dtype=getattr(config, "params_dtype", torch.bfloat16),
        router_dtype={"fp32": torch.float32, "fp64": torch.float64}.get(
            getattr(config, "moe_router_dtype", None), getattr(config, "params_dtype", torch.bfloat16)),
        aux_loss_coeff=getattr(config, "moe_aux_loss_coeff", 0.0) or 0.0,
        z_loss_coeff=getattr(config, "moe_z_loss_coeff", 0.0) or 0.0,
        norm_type="rmsnorm" if getattr(config, "normalization", "LayerNorm") == "RMSNorm" else "layernorm",
        norm_eps=getattr(config, "layernorm_epsilon", 1e-5),
    )


def _require_megatron():
    try:
        from megatron.core import parallel_state  # noqa: F401
        from megatron.core.transformer.module import MegatronModule  # noqa: F401
        from megatron.core.transformer.spec_utils import ModuleSpec  # noqa: F401
    except Exception as e:  # noqa: BLE001
        raise ImportError("megatron-core is required for the Megatron layer spec "
                          "(pip install megatron-core); the standalone TransformerLayer does not need it") from e


def build_fluid_transformer_layer_class():
    """Create the MegatronModule subclass lazily so that importing this module never needs Megatron."""
    _require_megatron()
    from megatron.core import parallel_state as mpu
    from megatron.core.transformer.module import MegatronModule

    class FluidTransformerLayer(MegatronModule):
        def __init__(self, config, submodules=None, layer_number: int = 1, pg_collection=None, vp_stage=None, **_):
            super().__init__(config=config)
            # groups from the collection Megatron hands over (fluid/layer/fluid_spec.py:43-46),
            # from the global parallel state when it passes none
            cp_group = getattr(pg_collection, "cp", None) or mpu.get_context_parallel_group()
            ep_group = getattr(pg_collection, "ep", None) or mpu.get_expert_model_parallel_group()
            self.layer_number = layer_number
            self.layer = TransformerLayer(cp_group=cp_group, ep_group=ep_group,
                                          device=torch.device("cuda", torch.cuda.current_device()),
                                          **layer_kwargs_from_config(config, layer_number))

        def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None, **kwargs):
            if isinstance(rotary_pos_emb, (tuple, list)):
                rotary_pos_emb = rotary_pos_emb[0]
            return self.layer(hidden_states, rotary_pos_emb), None

        def sharded_state_dict(self, prefix: str = "", sharded_offsets=(), metadata=None):
            return {prefix + "layer." + k: v for k, v in self.layer.state_dict().items()}

    return FluidTransformerLayer


def get_fluid_gpt_layer_spec():
    _require_megatron()
    from megatron.core.transformer.spec_utils import ModuleSpec
    return ModuleSpec(module=build_fluid_transformer_layer_class())


get_fluid_custom_layers = get_fluid_gpt_layer_spec
