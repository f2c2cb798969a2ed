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


CHUNK_KEYS = ("moe_combine_chunks", "moe_dispatch_chunks", "attn_proj_chunks", "attn_qkv_chunks")


def add_parallel_args(ap, chunks: bool = False) -> None:
    """The flags the reference's drivers share (tests/run_block_benchmark.py:188-196): listing the
    presets, the data / sequence / expert parallel sizes, and (``chunks``) the four chunk counts.
    A size left out follows from the world size; a chunk count left out keeps the tuned default."""
    ap.add_argument("--list-models", action="store_true", help="print the model presets and exit")
    ap.add_argument("--dp-size", type=int, default=None, help="data-parallel replicas (default: world / cp)")
    ap.add_argument("--cp-size", type=int, default=None, help="sequence-parallel ranks (default: ep, else world / dp)")
    ap.add_argument("--ep-size", type=int, default=None, help="expert-parallel ranks (must equal --cp-size)")
    if chunks:
        for key in CHUNK_KEYS:
            ap.add_argument("--" + key.replace("_", "-"), type=int, default=None)


def handle_list_models(args) -> bool:
    """Print the presets when ``--list-models`` was given; the caller then returns."""
    if not getattr(args, "list_models", False):
        return False
    from .model_configs import MODEL_CONFIGS
    for name, cfg in MODEL_CONFIGS.items():
        print(f"{name:28s} hidden {cfg['hidden_size']:5d}  heads {cfg['num_heads']}/{cfg['num_kv_heads']}  "
              f"ffn {cfg['ffn_hidden']:6d}  experts {cfg['num_experts']:3d} top-{cfg['top_k']}  "
              f"layers {cfg.get('num_layers', 2)}  seq {cfg.get('seq_len', cfg.get('seq_per_rank', 0))}")
    return True


def resolve_parallel_sizes(world: int, dp_size=None, cp_size=None, ep_size=None):
    """``(dp, cp)`` for a world of ``world`` ranks from whichever of the three sizes were given.
    Sequence and expert parallelism share their group, so they must agree, and dp x cp must be
    the world size."""
    if cp_size is not None and ep_size is not None and cp_size != ep_size:
        raise ValueError(f"--cp-size {cp_size} and --ep-size {ep_size} differ: the two share one group here")
    cp = cp_size or ep_size
    if cp is None:
        if dp_size is not None and world % dp_size != 0:
            raise ValueError(f"--dp-size {dp_size} does not divide the world size {world}")
        cp = world // (dp_size or 1)
    if cp <= 0 or world % cp != 0:
        raise ValueError(f"sequence / expert parallel size {cp} does not divide the world size {world}")
    dp = world // cp
    if dp_size is not None and dp_size != dp:
        raise ValueError(f"--dp-size {dp_size} x cp {cp} is not the world size {world}")
    return dp, cp


def apply_chunk_args(args, bench: dict) -> dict:
    """Chunk counts given on the command line replace the tuned defaults in ``bench``."""
    for key in CHUNK_KEYS:
        val = getattr(args, key, None)
        if val is not None:
            bench[key] = int(val)
    return bench


def setup(model: str, overrides: dict = None, comm_mode: str = "auto", heap_bytes: int = 4 << 30, args=None):
    """Process group, preset and parallel context.  ``args`` may carry ``dp_size / cp_size /
    ep_size`` from ``add_parallel_args``; without them every rank joins one sequence- and
    expert-parallel group."""
    device = init_distributed()
    cfg = get_model_config(model)
    cfg.update(overrides or {})
    world = dist.get_world_size() if dist.is_initialized() else 1
    _, cp = resolve_parallel_sizes(world, getattr(args, "dp_size", None), getattr(args, "cp_size", None),
                                   getattr(args, "ep_size", None))
    fused = comm_mode in ("auto", "fused") and device.type == "cuda" and cp > 1
    pc = init_parallel(ep_size=cp, device=device, symmetric_heap_bytes=heap_bytes if fused else 0)
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
