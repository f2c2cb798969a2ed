"""Profiler driver: run the block benchmark with a capture range around a few iterations.

    nsys profile --capture-range=cudaProfilerApi python -m fluidmoe_b200.tools.profile_capture ...
    python -m fluidmoe_b200.tools.profile_capture --model mixtral_8x7b --trace out.json

Warm-up iterations run outside the range; the captured iterations are bracketed by
``cudaProfilerStart`` / ``cudaProfilerStop`` (so an external profiler started with a
"capture range = profiler API" option records only them) and each carries an NVTX range
``iter_<n>``; ``FLUID_NVTX=1`` adds the per-region ranges of the layers.  Without an external
profiler, ``--trace`` writes a Chrome trace with the PyTorch profiler and ``--table`` a per-kernel
table.  The reference drives nsys the same way (tests/nsys_fluidmoe.py:52-160).
"""
from __future__ import annotations

import argparse
import contextlib
import os

import torch
import torch.distributed as dist

from ..parallel.scheduler import get_backward_scheduler
from ..utils import nvtx
from . import common
from .experiment_configs import get_block_benchmark_defaults


@contextlib.contextmanager
def capture_range(enabled: bool = True):
    """``cudaProfilerStart`` / ``cudaProfilerStop`` around the body (no-op without CUDA)."""
    use = enabled and torch.cuda.is_available()
    if use:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    try:
        yield
    finally:
        if use:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral_8x7b")
    ap.add_argument("--impl", default="fluidmoe-full", choices=["fluidmoe-f", "fluidmoe-fb", "fluidmoe-full"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--trace", default="", help="write a Chrome trace of the captured iterations here")
    ap.add_argument("--table", default="", help="write a per-kernel table of the captured iterations here")
    common.add_parallel_args(ap)
    args = ap.parse_args(argv)
    if common.handle_list_models(args):
        return
    os.environ.setdefault("FLUID_NVTX", "1")
    bench = get_block_benchmark_defaults()
    comm_mode = "a2a" if args.impl == "fluidmoe-f" else "auto"
    device, cfg, pc = common.setup(args.model, {"num_layers": args.layers} if args.layers else {}, comm_mode, args=args)
    model = common.build_model(cfg, bench, pc, device, comm_mode)
    x = common.make_input(cfg, pc, device)
    sched = get_backward_scheduler()
    if args.impl == "fluidmoe-f":
        sched.disable()
    else:
        sched.enable(device)
        sched.configure_allreduce(args.impl == "fluidmoe-full", pc.dp_cp_group, pc.expert_dp_group,
                                  bench.get("gap_budgets"), bench.get("shared_ar_bw"), bench.get("expert_ar_bw"))
        model.setup_ar_buffer()
    common.run_iters(model, x, args.warmup, pc)
    rank0 = (not dist.is_initialized()) or dist.get_rank() == 0
    prof = None
    if (args.trace or args.table) and rank0:
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if device.type == "cuda" else [])
        prof = profile(activities=acts)
    with capture_range(), (prof if prof is not None else contextlib.nullcontext()):
        for i in range(args.iters):
            with nvtx.nvtx_range(f"iter_{i}"):
                common.run_iters(model, x, 1, pc)
    if prof is not None:
        if args.trace:
            prof.export_chrome_trace(args.trace)
        if args.table:
            key = "self_cuda_time_total" if device.type == "cuda" else "self_cpu_time_total"
            with open(args.table, "w") as f:
                f.write(prof.key_averages().table(sort_by=key, row_limit=60))
    common.p0(f"captured {args.iters} iteration(s) of {args.impl} / {args.model}")
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
