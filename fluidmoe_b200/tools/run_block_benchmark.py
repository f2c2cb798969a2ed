"""Block benchmark: forward (inference) latency and training-iteration time of MoE transformer blocks.

    torchrun --nproc-per-node N -m fluidmoe_b200.tools.run_block_benchmark \
        --model cfg2_mixtral_moe_layer,cfg3_ulysses_attention_block,cfg23_mixtral_block --impl fluidmoe-full
    torchrun --nproc-per-node N -m fluidmoe_b200.tools.run_block_benchmark --model cfg23_mixtral_block --impl reference

``--impl``: ``fluidmoe-f`` (scheduler off, synchronous all-to-all: the baseline), ``fluidmoe-fb``
(deferred dW, one all-reduce at the end), ``fluidmoe-full`` (deferred dW + trickled all-reduce) and
``reference`` (the unmodified reference implementation from ``--ref-root``, full mode, in the
nearest configuration it can express: ``model_configs.reference_variant``).  ``--matched`` makes
this framework's arms run that same reference-expressible configuration.  Several presets can be
given; they run one after the other in the same process group.

For every preset one line is printed, in the format of the reference's
tests/run_block_benchmark.py:485-488 with two more fields::

    RESULT impl=... model=... gpus=N forward_ms=... iter_ms=... tokens_per_sec=... exposed_comm_ms=... exposed_comm_frac=...

``forward_ms`` is the forward pass under ``torch.no_grad()``; ``iter_ms`` forward + backward +
gradient reduction; both device-timed, maximum over ranks.  ``exposed_comm_ms`` (device-initiated
transport only) is the communication time per iteration the compute stream could not hide: waits
of gated GEMM producers, stand-alone wait kernels and the push kernels
(``FusedCommContext.comm_metrics``).  The reference's Megatron / DeepSpeed arms need those
packages (``tools.external_baselines``).
"""
from __future__ import annotations

import argparse
import gc
import os
import sys

import torch
import torch.distributed as dist

from ..parallel.scheduler import BackwardScheduler, get_backward_scheduler
from . import common
from .experiment_configs import get_block_benchmark_defaults
from .model_configs import get_model_config, reference_variant

IMPLS = ["fluidmoe-f", "fluidmoe-fb", "fluidmoe-full", "reference"]


def _result(impl, name, world, fwd_ms, iter_ms, tokens, metrics=None):
    line = (f"RESULT impl={impl} model={name} gpus={world} forward_ms={fwd_ms:.3f} iter_ms={iter_ms:.3f} "
            f"tokens_per_sec={tokens / (iter_ms / 1e3):.1f}")
    if metrics:
        line += (f" exposed_comm_ms={metrics['exposed_comm_ms']:.3f} exposed_comm_frac="
                 f"{metrics['exposed_comm_ms'] / max(iter_ms, 1e-9):.4f} gated_gemm_wait_ms={metrics['gated_gemm_wait_ms']:.3f}"
                 f" wait_kernels_ms={metrics['wait_kernels_ms']:.3f} push_kernels_ms={metrics['push_kernels_ms']:.3f}")
    common.p0(line)


def run_ours(name, cfg, args, device, pc, bench):
    comm_mode = "a2a" if args.impl == "fluidmoe-f" and args.comm == "auto" else args.comm
    BackwardScheduler.reset()
    model = common.build_model(cfg, bench, pc, device, comm_mode)
    x = common.make_input(cfg, pc, device)
    rotary = common.make_rotary(cfg, pc, device)
    model.prepare_chunk_status(x)          # warns once per region that falls back to fewer chunks
    sched = get_backward_scheduler()
    if args.impl == "fluidmoe-f":
        sched.disable()
    else:
        sched.enable(device)
    sched.configure_allreduce(args.impl == "fluidmoe-full", pc.dp_cp_group, pc.expert_dp_group,
                              bench.get("gap_budgets"), bench.get("shared_ar_bw"), bench.get("expert_ar_bw"))
    sched.eager_ar = pc.fused_ctx is not None and comm_mode in ("auto", "fused")
    if args.impl != "fluidmoe-f":
        model.setup_ar_buffer()
    common.run_iters(model, x, args.warmup, pc, rotary=rotary)
    common.run_iters(model, x, max(1, args.warmup // 2), pc, forward_only=True, rotary=rotary)
    fwd_ms = common.time_iters(model, x, args.iters, pc, forward_only=True, rotary=rotary)
    iter_ms = common.time_iters(model, x, args.iters, pc, rotary=rotary)
    metrics = None
    if pc.fused_ctx is not None and comm_mode in ("auto", "fused") and args.comm_metrics:
        pc.fused_ctx.enable_comm_metrics(True)
        common.run_iters(model, x, args.iters, pc, rotary=rotary)
        metrics = {k: v / args.iters for k, v in pc.fused_ctx.comm_metrics().items()}
        pc.fused_ctx.enable_comm_metrics(False)
        t = torch.tensor([metrics[k] for k in sorted(metrics)], dtype=torch.float64, device=device)
        if pc.world_size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        metrics = dict(zip(sorted(metrics), t.tolist()))
    tokens = x.shape[0] * x.shape[1] * max(1, pc.cp_size) * max(1, pc.dp_size)
    _result(args.impl + ("-matched" if args.matched else ""), name, pc.world_size, fwd_ms, iter_ms, tokens, metrics)
    del model, x
    if pc.fused_ctx is not None:
        pc.fused_ctx.release_all()
    BackwardScheduler.reset()


def run_reference(name, cfg, args, device, pc, bench):
    """The reference's own layer stack and scheduler (full mode), driven the way its
    tests/smoke_phase1.py:61-101 does, from an installed copy under ``--ref-root``."""
    ref_root = os.path.abspath(args.ref_root)
    if not os.path.isdir(os.path.join(ref_root, "fluid")):
        common.p0(f"RESULT impl=reference model={name} unavailable=no_reference_under_{ref_root}")
        return
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    mine = sys.modules.get("fluid")
    if mine is not None and not os.path.abspath(getattr(mine, "__file__", "")).startswith(ref_root):
        for k in [k for k in sys.modules if k == "fluid" or k.startswith("fluid.")]:
            del sys.modules[k]
    os.environ.setdefault("FLUIDMOE_P2P_BACKEND", "nccl")
    from fluid.core.scheduler import get_backward_scheduler as ref_sched_fn   # the reference package
    from fluid.layer.transformer import TransformerModel as RefModel
    world = pc.world_size
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29543")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    group = dist.new_group(list(range(world)))
    all_group = dist.new_group(list(range(world)))
    rc = reference_variant(cfg)
    torch.manual_seed(1234)
    model = RefModel(num_layers=int(rc.get("num_layers", 1)), hidden_size=int(rc["hidden_size"]),
                     num_heads=int(rc["num_heads"]), num_kv_heads=int(rc["num_kv_heads"]),
                     ffn_hidden_size=int(rc["ffn_hidden"]), num_experts=int(rc["num_experts"]), top_k=int(rc["top_k"]),
                     cp_group=group, ep_group=group, moe_combine_chunks=int(bench.get("moe_combine_chunks", 1)),
                     moe_dispatch_chunks=int(bench.get("moe_dispatch_chunks", 1)),
                     attn_proj_chunks=int(bench.get("attn_proj_chunks", 1)),
                     attn_qkv_chunks=int(bench.get("attn_qkv_chunks", 1)), capacity_factor=float(rc["capacity_factor"]),
                     dtype=torch.bfloat16, device=device, router_dtype=torch.float32)
    x = common.make_input(cfg, pc, device)
    rotary = common.make_rotary(dict(cfg, rope=True), pc, device).view(-1, 1, 1, int(rc["hidden_size"]) // int(rc["num_heads"]))
    model.prepare_chunk_status(x.detach())
    sched = ref_sched_fn()
    sched.enable()
    sched.configure_allreduce(enabled=True, shared_dp_group=all_group, expert_dp_group=None,
                              gap_budgets=bench.get("gap_budgets"), shared_ar_bw=bench.get("shared_ar_bw"),
                              expert_ar_bw=bench.get("expert_ar_bw"))
    model.setup_ar_buffer()
    params = list(model.parameters())

    def forward(inp):
        for layer in model.layers:
            inp = layer(inp, rotary)
        return inp

    def run(n, forward_only=False):
        for _ in range(n):
            if forward_only:
                with torch.no_grad():
                    forward(x)
                continue
            x.grad = None
            for p in params:
                p.grad = None
                if hasattr(p, "_ar_buf_written"):
                    p._ar_buf_written = False
            forward(x).sum().backward()
            sched.finish_batch()
            sched.clear_iteration()

    def timed(n, forward_only=False):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        run(n, forward_only)
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / n], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    run(args.warmup)
    run(max(1, args.warmup // 2), True)
    fwd_ms, iter_ms = timed(args.iters, True), timed(args.iters)
    tokens = x.shape[0] * x.shape[1] * world
    _result("reference", name, world, fwd_ms, iter_ms, tokens)
    del model, x
    gc.collect()
    torch.cuda.empty_cache()


def main(argv=None):
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "1")
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral_8x7b", help="preset name, or several separated by commas")
    ap.add_argument("--impl", default="fluidmoe-full", choices=IMPLS)
    ap.add_argument("--comm", default="auto", choices=["auto", "a2a", "p2p", "fused"])
    ap.add_argument("--matched", action="store_true",
                    help="run this framework's arm in the configuration the reference arm runs")
    ap.add_argument("--no-comm-metrics", dest="comm_metrics", action="store_false")
    ap.add_argument("--ref-root", default=os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__)))), "baseline", "_ref"))
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--iters", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--heap-gb", type=float, default=4.0)
    common.add_parallel_args(ap, chunks=True)
    args = ap.parse_args(argv)
    if common.handle_list_models(args):
        return
    bench = common.apply_chunk_args(args, get_block_benchmark_defaults())
    args.warmup = args.warmup if args.warmup is not None else bench["warmup"]
    args.iters = args.iters if args.iters is not None else bench["iters"]
    names = [n for n in args.model.split(",") if n]
    comm_mode = "a2a" if args.impl in ("fluidmoe-f", "reference") and args.comm == "auto" else args.comm
    device, _, pc = common.setup(names[0], None, comm_mode, heap_bytes=int(args.heap_gb * (1 << 30)), args=args)
    for name in names:
        cfg = get_model_config(name)
        if args.layers:
            cfg["num_layers"] = args.layers
        if args.matched and args.impl != "reference":
            cfg = reference_variant(cfg)
        if args.impl == "reference":
            run_reference(name, cfg, args, device, pc, bench)
        else:
            run_ours(name, cfg, args, device, pc, bench)
        gc.collect()
        if device.type == "cuda":
            torch.cuda.empty_cache()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
