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


def _writes_shards(ep_group) -> bool:
    """With data-parallel replicas of the expert-parallel group every replica holds the same shards:
    only the replica whose first member is global rank 0 writes them."""
    if not dist.is_initialized() or ep_group is None:
        return True
    return dist.get_global_rank(ep_group, 0) == 0


def save_checkpoint(model: torch.nn.Module, directory: str, ep_group=None, optimizer=None,
                    step: int = 0, extra: Optional[dict] = None) -> str:
    """One ``shard_epNNN.pt`` per expert-parallel rank (expert tensors, the rank's optimizer state;
    rank 0 also the dense tensors) and ``manifest.json``.  Only the first data-parallel replica
    writes; the closing barrier spans every rank of the job."""
    os.makedirs(directory, exist_ok=True)
    rank = dist.get_rank(ep_group) if dist.is_initialized() else 0
    world = dist.get_world_size(ep_group) if dist.is_initialized() else 1
    writer = _writes_shards(ep_group)
    sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    shard = {k: v for k, v in sd.items() if _is_expert_key(k) or rank == 0}
    payload = {"model": shard}
    if optimizer is not None:
        payload["optimizer"] = optimizer.state_dict()
        names = {id(p): n for n, p in model.named_parameters()}
        payload["optimizer_param_names"] = [names.get(id(p), "") for p in getattr(optimizer, "params", [])]
    if writer:
        torch.save(payload, os.path.join(directory, f"shard_ep{rank:03d}.pt"))
    if rank == 0 and writer:
        manifest = dict(format="fluidmoe_b200.sharded.v1", step=step, ep_size=world,
                        keys={k: dict(shape=list(v.shape), dtype=str(v.dtype), expert=_is_expert_key(k))
                              for k, v in sd.items()}, extra=extra or {})
        with open(os.path.join(directory, "manifest.json"), "w") as f:
            json.dump(manifest, f, indent=1)
    if dist.is_initialized():
        dist.barrier()
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
    payloads = [torch.load(os.path.join(directory, f"shard_ep{r:03d}.pt"), map_location="cpu") for r in range(old)]
    shards = [p["model"] for p in payloads]
    dense = {k: v for k, v in shards[0].items() if not _is_expert_key(k)}
    full = {k: torch.cat([s[k] for s in shards], dim=0) for k in shards[0] if _is_expert_key(k)}
    # optimizer state: expert moments are split along the expert dimension like the weights, every
    # other entry is replicated and taken from rank 0
    opt_parts = None
    if all("optimizer" in p for p in payloads):
        names = payloads[0].get("optimizer_param_names")
        if names is None:
            raise ValueError("checkpoint holds optimizer state without parameter names; it cannot be resharded")
        opt_parts = [dict(step=payloads[0]["optimizer"]["step"], state={}) for _ in range(new_ep_size)]
        for i, name in enumerate(names):
            per_rank = [p["optimizer"]["state"].get(i) for p in payloads]
            if not per_rank[0]:
                continue
            for r in range(new_ep_size):
                if _is_expert_key(name):
                    opt_parts[r]["state"][i] = {
                        k: (torch.cat([st[k] for st in per_rank], dim=0).chunk(new_ep_size, dim=0)[r].clone()
                            if torch.is_tensor(per_rank[0][k]) else per_rank[0][k]) for k in per_rank[0]}
                else:
                    opt_parts[r]["state"][i] = per_rank[0]
    elif any("optimizer" in p for p in payloads):
        raise ValueError("only some shards hold optimizer state")
    os.makedirs(out_directory, exist_ok=True)
    for r in range(new_ep_size):
        part = {k: v.chunk(new_ep_size, dim=0)[r].clone() for k, v in full.items()}
        if r == 0:
            part.update(dense)
        out = {"model": part}
        if opt_parts is not None:
            out["optimizer"] = opt_parts[r]
            out["optimizer_param_names"] = payloads[0]["optimizer_param_names"]
        torch.save(out, os.path.join(out_directory, f"shard_ep{r:03d}.pt"))
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
