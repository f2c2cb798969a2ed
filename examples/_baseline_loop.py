"""Shared training loop of the external-baseline examples (block stack on random activations)."""
from __future__ import annotations

import argparse
import time

import torch
import torch.distributed as dist

from fluidmoe_b200.distributed import init_distributed, init_parallel
from fluidmoe_b200.tools import external_baselines as eb
from fluidmoe_b200.tools.model_configs import get_model_config


def run(arm: str) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral_8x7b")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--lr", type=float, default=3e-4)
    args = ap.parse_args()
    try:
        if not eb.available()[arm]:
            eb._need(*(("megatron.core", "transformer_engine") if arm == "megatron" else ("deepspeed",)))
    except eb.BaselineUnavailable as e:
        print(f"{arm} baseline unavailable: {e}")
        return
    device = init_distributed()
    world = dist.get_world_size() if dist.is_initialized() else 1
    pc = init_parallel(ep_size=world, device=device)
    cfg = dict(get_model_config(args.model))
    if args.layers:
        cfg["num_layers"] = args.layers
    if arm == "megatron":
        model = eb.build_megatron_baseline(cfg, pc.cp_group, pc.ep_group, device=device)
    else:
        model = eb.build_deepspeed_ulysses_baseline(cfg, pc.cp_group, world, device=device)
    opt = torch.optim.AdamW(model.parameters(), lr=args.lr, fused=device.type == "cuda")
    s_local = cfg["seq_len"] // world
    x = torch.randn(s_local, cfg.get("batch_size", 1), cfg["hidden_size"], device=device, dtype=torch.bfloat16)
    for step in range(args.steps):
        t0 = time.perf_counter()
        out = model(x)
        out = out[0] if isinstance(out, tuple) else out
        out.float().pow(2).mean().backward()
        if world > 1:
            for p in model.parameters():
                if p.grad is not None and getattr(p, "allreduce", True):
                    g32 = p.grad.float()
                    dist.all_reduce(g32)
                    p.grad.copy_(g32 / world)
        opt.step()
        opt.zero_grad(set_to_none=True)
        if device.type == "cuda":
            torch.cuda.synchronize()
        if (not dist.is_initialized()) or dist.get_rank() == 0:
            print(f"step {step}: {(time.perf_counter() - t0) * 1e3:.1f} ms")
    if dist.is_initialized():
        dist.destroy_process_group()
