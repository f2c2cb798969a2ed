"""Autotuner (counterpart of the reference's tools/tune.py:172-472).

Step 1: greedy search of the per-region backward chunk counts over powers of two (stop when the
saving drops below ``min_saving_ms``), timing backward + ``finish_batch``.
Step 2a: all-reduce bandwidth sweep (the largest size gives the bytes/ms used for gap budgeting).
Step 2b: gap profiling: inter-all-to-all gaps per region, budget = p10 x 0.8.
Step 3 (device-initiated transport only, ``--comm fused``): the knobs that replace the gap model
there: the smallest slice the eager gradient reduction sends (``eager_ar_min_bytes``), the
reduction kernel (``grad_reduce``: library or two-shot over peer memory) and the CTA cap of the
weight-gradient side stream (``dw_side_ctas``, 0 = compute stream); each is kept only when it saves
at least ``min_saving_ms``.
Results are persisted with ``persist_block_benchmark_defaults`` (a JSON file; no source rewriting).
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from ..parallel.scheduler import BACKWARD_REGIONS, get_backward_scheduler
from . import common
from .experiment_configs import get_block_benchmark_defaults, get_tune_defaults, persist_block_benchmark_defaults

_CHUNK_KEYS = {"moe_combine": "moe_combine_chunks", "moe_dispatch": "moe_dispatch_chunks",
               "attn_proj": "attn_proj_chunks", "attn_qkv": "attn_qkv_chunks"}


def _time_config(cfg, bench, pc, device, comm, iters, warmup):
    model = common.build_model(cfg, bench, pc, device, comm)
    x = common.make_input(cfg, pc, device)
    sched = get_backward_scheduler()
    sched.enable(device)
    sched.configure_allreduce(False, pc.dp_cp_group, pc.expert_dp_group)
    model.setup_ar_buffer()
    common.run_iters(model, x, warmup, pc)
    ms = common.time_iters(model, x, iters, pc)
    del model
    return ms


def tune_chunks(cfg, bench, pc, device, comm, td) -> dict:
    best = dict(bench)
    for key in _CHUNK_KEYS.values():
        best[key] = 1
    best_ms = _time_config(cfg, best, pc, device, comm, td["iters"], td["warmup"])
    common.p0(f"[tune] all regions 1 chunk: {best_ms:.3f} ms")
    for region in BACKWARD_REGIONS:
        key = _CHUNK_KEYS[region]
        c = 2
        while c <= td["max_chunks"]:
            trial = dict(best)
            trial[key] = c
            ms = _time_config(cfg, trial, pc, device, comm, td["iters"], td["warmup"])
            common.p0(f"[tune] {region} chunks={c}: {ms:.3f} ms (best {best_ms:.3f})")
            if best_ms - ms < td["min_saving_ms"]:
                break
            best, best_ms = trial, ms
            c *= 2
    return {k: best[k] for k in _CHUNK_KEYS.values()}


def tune_allreduce(cfg, bench, pc, device, comm, td) -> dict:
    sched = get_backward_scheduler()
    bw = sched.measure_ar_bandwidth(pc.dp_cp_group, sizes_mb=td["ar_sizes_mb"], warmup=3, repeat=10)
    bytes_per_ms = bw["bw_GBps"][-1] * 1e9 / 1e3 if bw["bw_GBps"] else 0.0
    model = common.build_model(cfg, bench, pc, device, comm)
    x = common.make_input(cfg, pc, device)
    sched.enable(device)
    sched.configure_allreduce(False, pc.dp_cp_group, pc.expert_dp_group)
    model.setup_ar_buffer()
    common.run_iters(model, x, td["warmup"], pc)
    sched.profiling = True
    sched.reset_gap_times()
    common.run_iters(model, x, td["iters"], pc)
    gaps = sched.process_gap_events()
    sched.profiling = False
    budgets = {}
    for region in BACKWARD_REGIONS:
        vals = sorted(gaps.get(region, []))
        if vals:
            p = vals[max(0, int(len(vals) * td["gap_percentile"] / 100) - 1)]
            budgets[region] = max(0.0, p * td["gap_safety"])
    return dict(shared_ar_bw=bytes_per_ms, expert_ar_bw=bytes_per_ms, gap_budgets=budgets)


def _time_fused(cfg, bench, pc, device, td, eager_ar_min_bytes, grad_reduce, dw_side_ctas):
    from ..parallel.ddp import FluidDDP
    from ..parallel.scheduler import BackwardScheduler
    BackwardScheduler.reset()
    sched = get_backward_scheduler()
    sched.enable(device)
    model = common.build_model(cfg, bench, pc, device, "fused")
    x = common.make_input(cfg, pc, device)
    ddp = FluidDDP(None, model, sched, dp_cp_group=pc.dp_cp_group, expert_dp_group=pc.expert_dp_group,
                   grad_reduce=grad_reduce)
    sched.eager_ar_min_bytes = int(eager_ar_min_bytes)
    sched.dw_on_side_stream, sched.dw_max_ctas = dw_side_ctas > 0, dw_side_ctas
    common.run_iters(ddp.module, x, td["warmup"], pc)
    ms = common.time_iters(ddp.module, x, td["iters"], pc)
    del ddp, model
    if pc.fused_ctx is not None:
        pc.fused_ctx.release_all()
    return ms


def tune_fused(cfg, bench, pc, device, td) -> dict:
    best = dict(eager_ar_min_bytes=32 << 20, grad_reduce="nccl", dw_side_ctas=0)
    best_ms = _time_fused(cfg, bench, pc, device, td, **best)
    common.p0(f"[tune] fused defaults {best}: {best_ms:.3f} ms")
    trials = [("eager_ar_min_bytes", v) for v in (8 << 20, 128 << 20)] + [("grad_reduce", "symm")] + \
             [("dw_side_ctas", v) for v in td.get("side_ctas", (48,))]
    for key, val in trials:
        trial = dict(best, **{key: val})
        ms = _time_fused(cfg, bench, pc, device, td, **trial)
        common.p0(f"[tune] fused {key}={val}: {ms:.3f} ms (best {best_ms:.3f})")
        if best_ms - ms >= td["min_saving_ms"]:
            best, best_ms = trial, ms
    return {"fused_" + k: v for k, v in best.items()}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral_8x7b")
    ap.add_argument("--comm", default="p2p")
    ap.add_argument("--node-name", dest="node", default=None,
                    help="key under which the tuned values are stored (not --node: the launcher would take it for --node-rank)")
    ap.add_argument("--skip-chunks", action="store_true")
    common.add_parallel_args(ap)
    args = ap.parse_args(argv)
    if common.handle_list_models(args):
        return
    td = get_tune_defaults()
    bench = get_block_benchmark_defaults(args.node)
    device, cfg, pc = common.setup(args.model, None, args.comm, args=args)
    result = {}
    if not args.skip_chunks:
        result.update(tune_chunks(cfg, bench, pc, device, args.comm, td))
        bench.update(result)
    if args.comm in ("fused", "auto") and pc.fused_ctx is not None:
        result.update(tune_fused(cfg, bench, pc, device, td))
    else:
        result.update(tune_allreduce(cfg, bench, pc, device, args.comm, td))
    if not dist.is_initialized() or dist.get_rank() == 0:
        path = persist_block_benchmark_defaults(result, args.node)
        print(f"[tune] wrote {path}: {result}", flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
