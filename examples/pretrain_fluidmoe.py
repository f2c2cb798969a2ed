"""Train the MoE language model of this framework on synthetic or tokenised text data.

    torchrun --nproc-per-node N examples/pretrain_fluidmoe.py --layers 4 --steps 100

Sequence is split contiguously over the sequence-parallel group (rank r trains on positions
``[r*s_local, (r+1)*s_local)``), as the reference's example does for its Megatron run
(examples/pretrain_fluidmoe.py:97-117).  ``--data`` takes a ``.npy`` / ``.bin`` file of token ids
(see ``examples/text_dataset.py``); without it random ids are used.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fluidmoe_b200.distributed import init_distributed, init_parallel  # noqa: E402
from fluidmoe_b200.models.gpt import MoEGPT  # noqa: E402
from fluidmoe_b200.ops.optim import FusedAdam  # noqa: E402
from fluidmoe_b200.parallel.ddp import FluidDDP, FluidOptimizerWrapper  # noqa: E402
from fluidmoe_b200.parallel.scheduler import get_backward_scheduler  # noqa: E402
from fluidmoe_b200.utils.checkpoint import load_checkpoint, save_checkpoint  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=2048, help="positions per rank")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--data", default=os.environ.get("FLUIDMOE_DATASET_SOURCE", ""))
    ap.add_argument("--save", default="")
    ap.add_argument("--load", default="")
    ap.add_argument("--save-interval", type=int, default=0)
    args = ap.parse_args()

    device = init_distributed()
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    pc = init_parallel(ep_size=world, device=device,
                       symmetric_heap_bytes=(4 << 30) if (world > 1 and device.type == "cuda") else 0)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    model = MoEGPT(args.vocab, args.layers, args.hidden, args.heads, args.kv_heads, args.ffn, args.experts,
                   args.top_k, pc.cp_group, pc.ep_group, dtype=dtype, device=device, router_dtype=torch.float32,
                   activation_func="swiglu", norm_type="rmsnorm", moe_combine_chunks=2, moe_dispatch_chunks=2,
                   attn_proj_chunks=2, attn_qkv_chunks=2, parallel_ctx=pc)
    sched = get_backward_scheduler()
    sched.enable(device)
    ddp = FluidDDP(None, model, sched, dp_cp_group=pc.dp_cp_group, expert_dp_group=pc.expert_dp_group)
    opt = FluidOptimizerWrapper(FusedAdam(model.parameters(), lr=args.lr), sched)
    if args.load:
        load_checkpoint(model, args.load, pc.ep_group, optimizer=opt.optimizer)
    if args.data:
        from text_dataset import TokenFileDataset
        data = TokenFileDataset(args.data, args.seq * world + 1)
    else:
        data = None
    gen = torch.Generator().manual_seed(1234)
    for step in range(1, args.steps + 1):
        if data is not None:
            full = data[step % len(data)].view(-1, 1).expand(-1, args.batch)
        else:
            full = torch.randint(0, args.vocab, (args.seq * world + 1, args.batch), generator=gen)
        ids = full[rank * args.seq:(rank + 1) * args.seq + 1].to(device)
        t0 = time.perf_counter()
        ddp.zero_grad_buffer()
        loss = ddp(ids[:-1], ids[1:])
        loss.backward()
        ddp.finish_grad_sync()
        opt.step()
        lv = loss.detach().clone()
        if world > 1:
            dist.all_reduce(lv)
            lv /= world
        if rank == 0:
            print(f" iteration {step:6d}/{args.steps} | elapsed time per iteration (ms): "
                  f"{(time.perf_counter() - t0) * 1e3:.1f} | lm loss: {lv.item():.6E}", flush=True)
        if args.save and args.save_interval and step % args.save_interval == 0:
            save_checkpoint(model, args.save, pc.ep_group, optimizer=opt.optimizer, step=step)
    if args.save:
        save_checkpoint(model, args.save, pc.ep_group, optimizer=opt.optimizer, step=args.steps)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
