"""Sharded checkpoints: one file per expert-parallel rank plus a JSON manifest.

The state-dict keys and tensor layouts are those of the reference layer
(fluid/layer/transformer.py:902-956): ``ln{1,2}_weight/bias [H]``, ``qkv_weight [n_kv*(q/kv+2)*d, H]``
(rows grouped per KV group as q.., k, v), ``proj_weight [H, n_h*d]``, ``router_weight [H, E]``,
``moe_w1 [nle, H, F]`` and ``moe_w2 [nle, F, H]`` sharded over the expert-parallel group.  Extensions:
SwiGLU stores ``moe_w1 [nle, H, 2F]`` (gate half first), RMSNorm has no bias keys, shared experts add
``shared_w1 [H, n_sh*F(*2)]`` / ``shared_w2 [n_sh*F, H]``.  Dense tensors are written by rank 0 of
the group only; expert tensors by every rank.  Scheduler and gradient buffers are not saved.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

EXPERT_KEYS = ("moe_w1", "moe_w2")


def _is_expert_key(key: str) -> bool:
    return key.rsplit(".", 1)[-1] in EXPERT_KEYS


def save_checkpoint(model: torch.nn.Module, directory: str, ep_group=None, optimizer=None,
                    step: int = 0, extra: Optional[dict] = None) -> str:
    os.makedirs(directory, exist_ok=True)
    rank = dist.get_rank(ep_group) if dist.is_initialized() else 0
    world = dist.get_world_size(ep_group) if dist.is_initialized() else 1
    sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    shard = {k: v for k, v in sd.items() if _is_expert_key(k) or rank == 0}
    payload = {"model": shard}
    if optimizer is not None:
        payload["optimizer"] = optimizer.state_dict()
    torch.save(payload, os.path.join(directory, f"shard_ep{rank:03d}.pt"))
    if rank == 0:
        manifest = dict(format="fluidmoe_b200.sharded.v1", step=step, ep_size=world,
                        keys={k: dict(shape=list(v.shape), dtype=str(v.dtype), expert=_is_expert_key(k))
                              for k, v in sd.items()}, extra=extra or {})
        with open(os.path.join(directory, "manifest.json"), "w") as f:
            json.dump(manifest, f, indent=1)
    if dist.is_initialized():
        dist.barrier(group=ep_group)
    return directory


def load_checkpoint(model: torch.nn.Module, directory: str, ep_group=None, optimizer=None,
                    strict: bool = True) -> dict:
    rank = dist.get_rank(ep_group) if dist.is_initialized() else 0
    with open(os.path.join(directory, "manifest.json")) as f:
        manifest = json.load(f)
    world = dist.get_world_size(ep_group) if dist.is_initialized() else 1
    if manifest["ep_size"] != world:
        raise ValueError(f"checkpoint was written with ep_size={manifest['ep_size']}, this run has {world}; "
                         "use reshard_experts() first")
    own = torch.load(os.path.join(directory, f"shard_ep{rank:03d}.pt"), map_location="cpu")
    state: Dict[str, torch.Tensor] = dict(own["model"])
    if rank != 0:
        dense = torch.load(os.path.join(directory, "shard_ep000.pt"), map_location="cpu")["model"]
        state.update({k: v for k, v in dense.items() if not _is_expert_key(k)})
    model.load_state_dict(state, strict=strict)
    if optimizer is not None and "optimizer" in own:
        optimizer.load_state_dict(own["optimizer"])
    return manifest


def reshard_experts(directory: str, out_directory: str, new_ep_size: int) -> None:
    """Rewrite a checkpoint for another expert-parallel size (host-side, single process)."""
    with open(os.path.join(directory, "manifest.json")) as f:
        manifest = json.load(f)
    old = manifest["ep_size"]
    shards = [torch.load(os.path.join(directory, f"shard_ep{r:03d}.pt"), map_location="cpu")["model"] for r in range(old)]
    dense = {k: v for k, v in shards[0].items() if not _is_expert_key(k)}
    full = {k: torch.cat([s[k] for s in shards], dim=0) for k in shards[0] if _is_expert_key(k)}
    os.makedirs(out_directory, exist_ok=True)
    for r in range(new_ep_size):
        part = {k: v.chunk(new_ep_size, dim=0)[r].clone() for k, v in full.items()}
        if r == 0:
            part.update(dense)
        torch.save({"model": part}, os.path.join(out_directory, f"shard_ep{r:03d}.pt"))
    manifest["ep_size"] = new_ep_size
    with open(os.path.join(out_directory, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)


def load_reference_state_dict(model: torch.nn.Module, state_dict: Dict[str, torch.Tensor], strict: bool = True):
    """Load a state dict produced by the reference layer / model.  Keys written by its
    Transformer-Engine variant (``te_qkv_linear.weight``, ``te_proj_linear.weight``) are renamed;
    TE ``_extra_state`` entries are dropped."""
    out = {}
    for k, v in state_dict.items():
        if k.endswith("_extra_state"):
            continue
        k = k.replace("te_qkv_linear.weight", "qkv_weight").replace("te_proj_linear.weight", "proj_weight")
        out[k] = v
    return model.load_state_dict(out, strict=strict)
