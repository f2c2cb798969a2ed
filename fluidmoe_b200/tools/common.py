"""Shared helpers of the benchmark / tuning drivers: groups, model construction, timed iterations."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..distributed import init_distributed, init_parallel
from ..models.transformer import TransformerModel
from ..parallel.scheduler import get_backward_scheduler
from .model_configs import get_model_config


def p0(*a):
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(*a, flush=True)


def setup(model: str, overrides: dict = None, comm_mode: str = "auto", heap_bytes: int = 4 << 30):
    device = init_distributed()
    cfg = get_model_config(model)
    cfg.update(overrides or {})
    world = dist.get_world_size() if dist.is_initialized() else 1
    fused = comm_mode in ("auto", "fused") and device.type == "cuda" and world > 1
    pc = init_parallel(ep_size=world, device=device, symmetric_heap_bytes=heap_bytes if fused else 0)
    return device, cfg, pc


def zipf_logit_prior(num_experts: int, s: float, device) -> torch.Tensor:
    """Log of a Zipf(s) distribution over the experts: added to the router logits it makes expert
    e's selection probability fall like ``1 / (e + 1)^s``."""
    ranks = torch.arange(1, num_experts + 1, dtype=torch.float32, device=device)
    return torch.log(ranks.pow(-s) / ranks.pow(-s).sum())


def build_model(cfg: dict, bench: dict, pc, device, comm_mode: str = "auto", dtype=torch.bfloat16):
    model = _build_model(cfg, bench, pc, device, comm_mode, dtype)
    if float(cfg.get("zipf_s", 0.0)) > 0.0:
        prior = zipf_logit_prior(int(cfg["num_experts"]), float(cfg["zipf_s"]), device)
        for layer in model.layers:
            layer.set_router_bias(prior)
    return model


def make_rotary(cfg: dict, pc, device):
    """RoPE angles of the full sequence for presets that ask for it (``rope=True``), else None."""
    if not cfg.get("rope", False):
        return None
    from ..ops.rope import make_rope_freqs
    s_loc = seq_per_rank(cfg, pc)
    d = int(cfg["hidden_size"]) // int(cfg["num_heads"])
    return make_rope_freqs(s_loc * max(1, pc.cp_size), d, device=device)


def seq_per_rank(cfg: dict, pc) -> int:
    if "seq_per_rank" in cfg:
        return int(cfg["seq_per_rank"])
    return int(cfg["seq_len"]) // max(1, pc.cp_size)


def _build_model(cfg: dict, bench: dict, pc, device, comm_mode: str = "auto", dtype=torch.bfloat16):
    return TransformerModel(
        num_layers=int(cfg.get("num_layers", 2)), hidden_size=int(cfg["hidden_size"]),
        num_heads=int(cfg["num_heads"]), num_kv_heads=int(cfg["num_kv_heads"]),
        ffn_hidden_size=int(cfg["ffn_hidden"]), num_experts=int(cfg["num_experts"]), top_k=int(cfg["top_k"]),
        cp_group=pc.cp_group, ep_group=pc.ep_group,
        moe_combine_chunks=int(bench.get("moe_combine_chunks", 1)),
        moe_dispatch_chunks=int(bench.get("moe_dispatch_chunks", 1)),
        attn_proj_chunks=int(bench.get("attn_proj_chunks", 1)), attn_qkv_chunks=int(bench.get("attn_qkv_chunks", 1)),
        activation_func=cfg.get("activation", "gelu"), capacity_factor=float(cfg.get("capacity_factor", 1.0)),
        dtype=dtype, device=device, router_dtype=torch.float32, norm_type=cfg.get("norm_type", "layernorm"),
        num_shared_experts=int(cfg.get("num_shared_experts", 0)), comm_mode=comm_mode, parallel_ctx=pc,
        has_attention=bool(cfg.get("has_attention", True)), has_moe=bool(cfg.get("has_moe", True)))


def make_input(cfg: dict, pc, device, dtype=torch.bfloat16):
    s_loc = seq_per_rank(cfg, pc)
    x = torch.randn(s_loc, int(cfg["batch_size"]), int(cfg["hidden_size"]), dtype=dtype, device=device)
    return x.requires_grad_(True)


def run_iters(model, x, n: int, pc=None, forward_only: bool = False, rotary=None):
    sched = get_backward_scheduler()
    for _ in range(n):
        if forward_only:
            with torch.no_grad():
                model(x, rotary)
            continue
        x.grad = None
        for p in model.parameters():
            p.grad = None
            if hasattr(p, "_ar_buf_written"):
                p._ar_buf_written = False
        model(x, rotary).sum().backward()
        sched.finish_batch()
        if pc is not None and pc.fused_ctx is not None:
            pc.fused_ctx.iteration_barrier()
        sched.clear_iteration()


def time_iters(model, x, n: int, pc=None, forward_only: bool = False, rotary=None) -> float:
    """ms per iteration, device-timed, MAX over ranks."""
    cuda = x.is_cuda
    if cuda:
        torch.cuda.synchronize()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        run_iters(model, x, n, pc, forward_only, rotary)
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / n
    else:
        import time
        t0 = time.perf_counter()
        run_iters(model, x, n, pc, forward_only, rotary)
        ms = (time.perf_counter() - t0) * 1e3 / n
    t = torch.tensor([ms], dtype=torch.float64, device=x.device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()
