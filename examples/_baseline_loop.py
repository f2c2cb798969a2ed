"""Training loop of the external-baseline examples: the same language-model harness, data and log
format as ``pretrain_fluidmoe.py`` around a block stack built from another framework."""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import lm_harness as H  # noqa: E402
from fluidmoe_b200.distributed import init_distributed, init_parallel  # noqa: E402
from fluidmoe_b200.tools import external_baselines as eb  # noqa: E402


def preset_from_args(args) -> dict:
    """The keys ``tools.external_baselines`` reads, from the common command line."""
    return dict(hidden_size=args.hidden, num_heads=args.heads, num_kv_heads=args.kv_heads, ffn_hidden=args.ffn,
                num_experts=args.experts, top_k=args.top_k, num_layers=args.layers, capacity_factor=1.0,
                activation=args.activation, norm_type=args.norm)


def parse(extra=None):
    ap = argparse.ArgumentParser()
    H.add_common_args(ap)
    ap.add_argument("--activation", default="gelu", choices=["gelu", "swiglu"])
    ap.add_argument("--norm", default="layernorm", choices=["layernorm", "rmsnorm"])
    if extra is not None:
        extra(ap)
    return ap.parse_args()


def train(args, build_blocks, wrap_engine=None, arm: str = "baseline") -> None:
    """``build_blocks(cfg, pc, device)`` returns the block stack; ``wrap_engine(model, args)`` may
    return ``(engine, step_fn)`` to let another framework own backward and the optimizer."""
    device = init_distributed()
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    pc = init_parallel(ep_size=world, device=device)
    torch.manual_seed(args.seed)
    try:
        blocks = build_blocks(preset_from_args(args), pc, device)
    except eb.BaselineUnavailable as e:
        if rank == 0:
            print(f"{arm} baseline unavailable: {e}")
        return
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    model = H.BlockLM(blocks, args.vocab, args.hidden, dtype, device)
    params = [p for p in model.parameters() if p.requires_grad]
    engine_step = None
    if wrap_engine is not None:
        model, engine_step = wrap_engine(model, args)
    opt = None if engine_step else torch.optim.AdamW(params, lr=args.lr, weight_decay=0.0,
                                                     fused=device.type == "cuda")
    data = H.batches(args, rank, world, device)
    for step in range(1, args.steps + 1):
        t0 = time.perf_counter()
        ids = next(data)
        loss = model(ids[:-1], ids[1:])
        if engine_step is not None:
            engine_step(loss)
            gnorm = None
        else:
            loss.backward()
            if world > 1:       # fp32 reduction of replicated parameters; expert shards stay local
                for p in params:
                    if p.grad is not None and getattr(p, "allreduce", True):
                        g32 = p.grad.float()
                        dist.all_reduce(g32)
                        p.grad.copy_(g32 / world)
            gnorm = H.grad_norm(params, pc.ep_group) if step % args.log_interval == 0 else None
            opt.step()
            opt.zero_grad(set_to_none=True)
        if step % args.log_interval == 0:
            lv = H.mean_over_ranks(loss)
            if device.type == "cuda":
                torch.cuda.synchronize()
            if rank == 0:
                print(H.log_line(step, args.steps, (time.perf_counter() - t0) * 1e3, lv, gnorm, args.lr), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
