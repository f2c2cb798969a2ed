"""Block benchmark: forward and training-iteration time of a stack of MoE transformer blocks.

    torchrun --nproc-per-node N -m fluidmoe_b200.tools.run_block_benchmark --model mixtral_8x7b \
        --impl fluidmoe-full

``--impl``: ``fluidmoe-f`` (scheduler off, synchronous all-to-all: the baseline), ``fluidmoe-fb``
(deferred dW, one all-reduce at the end), ``fluidmoe-full`` (deferred dW + trickled all-reduce).
Prints ``RESULT impl=... forward_ms=... iter_ms=... tokens_per_sec=...`` like the reference's
tests/run_block_benchmark.py:485-488 (its Megatron / DeepSpeed arms need those packages and are not
reproduced here).
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from ..parallel.scheduler import get_backward_scheduler
from . import common
from .experiment_configs import get_block_benchmark_defaults


def main(argv=None):
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "1")
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral_8x7b")
    ap.add_argument("--impl", default="fluidmoe-full", choices=["fluidmoe-f", "fluidmoe-fb", "fluidmoe-full"])
    ap.add_argument("--comm", default="auto", choices=["auto", "a2a", "p2p", "fused"])
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--iters", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None)
    args = ap.parse_args(argv)
    bench = get_block_benchmark_defaults()
    overrides = {"num_layers": args.layers} if args.layers else {}
    comm_mode = "a2a" if args.impl == "fluidmoe-f" and args.comm == "auto" else args.comm
    device, cfg, pc = common.setup(args.model, overrides, comm_mode)
    model = common.build_model(cfg, bench, pc, device, comm_mode)
    x = common.make_input(cfg, pc, device)
    chunk_status = model.prepare_chunk_status(x)     # warns once per region that falls back
    sched = get_backward_scheduler()
    if args.impl == "fluidmoe-f":
        sched.disable()
    else:
        sched.enable(device)
    sched.configure_allreduce(args.impl == "fluidmoe-full", pc.dp_cp_group, pc.expert_dp_group,
                              bench.get("gap_budgets"), bench.get("shared_ar_bw"), bench.get("expert_ar_bw"))
    if args.impl != "fluidmoe-f":
        model.setup_ar_buffer()
    warmup = args.warmup if args.warmup is not None else bench["warmup"]
    iters = args.iters if args.iters is not None else bench["iters"]
    common.run_iters(model, x, warmup, pc)
    fwd_ms = common.time_iters(model, x, iters, pc, forward_only=True)
    iter_ms = common.time_iters(model, x, iters, pc)
    tokens = x.shape[0] * x.shape[1] * max(1, pc.cp_size) * max(1, pc.dp_size)
    common.p0(f"RESULT impl={args.impl} model={args.model} gpus={pc.world_size} forward_ms={fwd_ms:.3f} "
              f"iter_ms={iter_ms:.3f} tokens_per_sec={tokens / (iter_ms / 1e3):.1f}")
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
