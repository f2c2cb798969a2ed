"""Train the MoE language model of this framework on synthetic or tokenised text data.

    torchrun --nproc-per-node N examples/pretrain_fluidmoe.py --layers 4 --steps 100
    python examples/pretrain_fluidmoe.py --steps 5                      # one process (CPU or GPU)

The sequence is split contiguously over the sequence-parallel group, as the reference's example
does for its Megatron run (examples/pretrain_fluidmoe.py:97-117).  ``--data`` takes a token file
(see ``examples/text_dataset.py``); without it uniform random ids are used.  ``--comm`` picks the
transport (``auto``: device-initiated kernels when the GPUs can reach each other, else pairwise
overlap), ``--mode`` the scheduler mode (``F`` off, ``FB`` deferred weight gradients, ``full`` with
the trickled gradient reduction), ``--arch matched`` the reference's own architecture (GELU
experts, LayerNorm).  Every step prints one line in the Megatron log format (``lm loss``, ``grad
norm``, iteration time) that ``examples/run_training.sh`` parses; ``--micro-batches`` accumulates
several micro-batches per optimizer step (all but the last inside ``ddp.no_sync()``).
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import lm_harness as H  # noqa: E402
from fluidmoe_b200.distributed import init_distributed, init_parallel  # noqa: E402
from fluidmoe_b200.models.gpt import MoEGPT  # noqa: E402
from fluidmoe_b200.ops.optim import FusedAdam  # noqa: E402
from fluidmoe_b200.parallel.ddp import FluidDDP, FluidOptimizerWrapper  # noqa: E402
from fluidmoe_b200.parallel.scheduler import get_backward_scheduler  # noqa: E402
from fluidmoe_b200.utils.checkpoint import load_checkpoint, save_checkpoint  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    H.add_common_args(ap)
    ap.add_argument("--comm", default="auto", choices=["auto", "a2a", "p2p", "fused"])
    ap.add_argument("--mode", default="full", choices=["F", "FB", "full"])
    ap.add_argument("--arch", default="native", choices=["native", "matched"])
    ap.add_argument("--chunks", type=int, default=2)
    ap.add_argument("--micro-batches", type=int, default=1)
    ap.add_argument("--grad-reduce", default=None, choices=[None, "nccl", "symm"])
    ap.add_argument("--save", default="")
    ap.add_argument("--load", default="")
    ap.add_argument("--save-interval", type=int, default=0)
    args = ap.parse_args(argv)

    device = init_distributed()
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    fused = world > 1 and device.type == "cuda" and args.comm in ("auto", "fused")
    pc = init_parallel(ep_size=world, device=device, symmetric_heap_bytes=(4 << 30) if fused else 0)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    act, norm = ("gelu", "layernorm") if args.arch == "matched" else ("swiglu", "rmsnorm")
    torch.manual_seed(args.seed)
    model = MoEGPT(args.vocab, args.layers, args.hidden, args.heads, args.kv_heads, args.ffn, args.experts,
                   args.top_k, pc.cp_group, pc.ep_group, dtype=dtype, device=device, router_dtype=torch.float32,
                   activation_func=act, norm_type=norm, moe_combine_chunks=args.chunks,
                   moe_dispatch_chunks=args.chunks, attn_proj_chunks=args.chunks, attn_qkv_chunks=args.chunks,
                   comm_mode=args.comm, parallel_ctx=pc)
    sched = get_backward_scheduler()
    if args.mode == "F":
        sched.disable()
    else:
        sched.enable(device)
    ddp = FluidDDP(None, model, sched, dp_cp_group=pc.dp_cp_group, expert_dp_group=pc.expert_dp_group,
                   ar_enabled=args.mode == "full", grad_reduce=args.grad_reduce)
    opt = FluidOptimizerWrapper(FusedAdam(model.parameters(), lr=args.lr), sched)
    if args.load:
        load_checkpoint(model, args.load, pc.ep_group, optimizer=opt.optimizer)
    data = H.batches(args, rank, world, device)
    params = list(model.parameters())
    for step in range(1, args.steps + 1):
        t0 = time.perf_counter()
        ddp.zero_grad_buffer()
        loss_sum = torch.zeros((), device=device)
        for mb in range(args.micro_batches):
            ids = next(data)
            if mb < args.micro_batches - 1:
                with ddp.no_sync():
                    loss = ddp(ids[:-1], ids[1:]) / args.micro_batches
                    loss.backward()
            else:
                loss = ddp(ids[:-1], ids[1:]) / args.micro_batches
                loss.backward()
            loss_sum += loss.detach().float()
        ddp.finish_grad_sync()
        gnorm = H.grad_norm(params, pc.ep_group) if step % args.log_interval == 0 else None
        opt.step()
        if step % args.log_interval == 0:
            lv = H.mean_over_ranks(loss_sum)
            if device.type == "cuda":
                torch.cuda.synchronize()
            if rank == 0:
                print(H.log_line(step, args.steps, (time.perf_counter() - t0) * 1e3, lv, gnorm, args.lr), flush=True)
        if args.save and args.save_interval and step % args.save_interval == 0:
            save_checkpoint(model, args.save, pc.ep_group, optimizer=opt.optimizer, step=step)
    if args.save:
        save_checkpoint(model, args.save, pc.ep_group, optimizer=opt.optimizer, step=args.steps)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
