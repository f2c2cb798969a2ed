"""Exposed-communication report, MAX over ranks (counterpart of the reference's
tests/overlap_ratio_analyzer.py:43-182).

Host-submitted transports (``--comm p2p`` / ``a2a``): total vs visible all-to-all and all-reduce
time per region, from the scheduler's event pairs.  Device-initiated transport (``--comm fused`` /
``auto`` with a symmetric heap): there are no host-submitted all-to-alls to bracket; the report is
the time the compute stream could not hide, from the counters inside the kernels
(``FusedCommContext.comm_metrics``: waits of the gated GEMM producers, stand-alone wait kernels,
push kernels), next to the iteration time.
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from ..parallel.scheduler import get_backward_scheduler
from . import common
from .experiment_configs import get_block_benchmark_defaults


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral_8x7b")
    ap.add_argument("--comm", default="p2p")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--mode", choices=["sync", "interleaved"], default="interleaved",
                    help="interleaved: gradient reductions are trickled into the backward pass; "
                         "sync: they all run at its end")
    ap.add_argument("--num-layers", type=int, default=None, help="override the preset's layer count")
    common.add_parallel_args(ap)
    args = ap.parse_args(argv)
    if common.handle_list_models(args):
        return
    bench = get_block_benchmark_defaults()
    device, cfg, pc = common.setup(args.model, {"num_layers": args.num_layers} if args.num_layers else None,
                                   args.comm, args=args)
    model = common.build_model(cfg, bench, pc, device, args.comm)
    x = common.make_input(cfg, pc, device)
    sched = get_backward_scheduler()
    sched.enable(device)
    sched.configure_allreduce(True, pc.dp_cp_group, pc.expert_dp_group, bench.get("gap_budgets"),
                              bench.get("shared_ar_bw"), bench.get("expert_ar_bw"))
    model.setup_ar_buffer()
    if args.mode == "sync":
        sched.ar_enabled = False      # nothing is reduced inside the backward pass (tests/overlap_ratio_analyzer.py:137)
    rotary = common.make_rotary(cfg, pc, device)
    common.run_iters(model, x, args.warmup, pc, rotary=rotary)
    if pc.fused_ctx is not None and args.comm in ("auto", "fused"):
        sched.eager_ar = True
        iter_ms = common.time_iters(model, x, args.iters, pc, rotary=rotary)
        pc.fused_ctx.enable_comm_metrics(True)
        common.run_iters(model, x, args.iters, pc, rotary=rotary)
        m = pc.fused_ctx.comm_metrics()
        pc.fused_ctx.enable_comm_metrics(False)
        keys = sorted(m)
        vals = torch.tensor([m[k] / args.iters for k in keys], dtype=torch.float64, device=device)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        m = dict(zip(keys, vals.tolist()))
        common.p0(f"iter_ms={iter_ms:.3f} exposed_comm_ms={m['exposed_comm_ms']:.3f} "
                  f"exposed_comm_frac={m['exposed_comm_ms'] / max(iter_ms, 1e-9):.4f}")
        common.p0(f"  gated_gemm_wait_ms={m['gated_gemm_wait_ms']:.3f} wait_kernels_ms={m['wait_kernels_ms']:.3f} "
                  f"push_kernels_ms={m['push_kernels_ms']:.3f}")
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
        return
    sched.set_comm_metrics_enabled(True)
    sched.reset_comm_metrics()
    common.run_iters(model, x, args.iters, pc)
    m = sched.get_comm_metrics()
    sched.set_comm_metrics_enabled(False)
    vals = torch.tensor([m["a2a_total_ms"], m["a2a_visible_ms"], m["ar_total_ms"], m["ar_visible_ms"]],
                        dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    a2a_t, a2a_v, ar_t, ar_v = (v / args.iters for v in vals.tolist())
    common.p0(f"a2a_total_ms={a2a_t:.3f} a2a_visible_ms={a2a_v:.3f} a2a_overlap={1 - a2a_v / a2a_t if a2a_t > 0 else 0:.3f}")
    common.p0(f"ar_total_ms={ar_t:.3f} ar_visible_ms={ar_v:.3f} ar_overlap={1 - ar_v / ar_t if ar_t > 0 else 0:.3f}")
    for region, b in sorted(m["per_region"].items()):
        common.p0(f"  {region:14s} a2a {b['a2a_total_ms'] / args.iters:8.3f} ms visible {b['a2a_visible_ms'] / args.iters:8.3f} ms")
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
