"""Transport micro-benchmark with data-integrity check: NCCL all-to-all, NCCL pairwise in
round-robin order, and this library's device-initiated all-to-all over symmetric memory.

Every transport first moves a pattern derived from (sender, receiver, index) and must reproduce it
bit for bit before it is timed (as in the reference's tests/bench_comm.py:57-93).
    torchrun --nproc-per-node N -m fluidmoe_b200.tools.bench_comm --sizes-mib 1 8 32

``--allreduce`` times the gradient all-reduce instead: the library collective against this
library's two-shot kernel over peer memory (``SymmGradReducer``: the form the scheduler calls, on
slices of a flat fp32 buffer), each checked against the other before it is timed; sizes are the
slice sizes in MiB.  Bus bandwidth is ``2 (P-1)/P * bytes / time``.
    torchrun --nproc-per-node N -m fluidmoe_b200.tools.bench_comm --allreduce --sizes-mib 32 128 512
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from ..distributed import init_distributed
from ..parallel.schedule import partner_table
from . import common


def _pattern(rank, world, n, device):
    idx = torch.arange(n, device=device, dtype=torch.int32)
    return torch.stack([(rank * 1000003 + p * 7919) + idx for p in range(world)]).contiguous()


def _check(out, rank, world, n, device, name):
    idx = torch.arange(n, device=device, dtype=torch.int32)
    for p in range(world):
        if not torch.equal(out[p], (p * 1000003 + rank * 7919) + idx):
            raise AssertionError(f"{name}: data from rank {p} is corrupt on rank {rank}")


_ITERS, _WARMUP = 20, 5     # replaced by --iters / --warmup


def _time(fn, iters=None, warmup=None):
    iters = _ITERS if iters is None else iters
    warmup = _WARMUP if warmup is None else warmup
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def bench_allreduce(args, device, rank, world):
    from ..parallel.symm import SymmGradReducer, SymmetricHeap
    biggest = int(max(args.sizes_mib) * (1 << 20))
    heap = SymmetricHeap(None, biggest + (64 << 20), device)
    for ctas in args.ctas:
        red = SymmGradReducer(heap, num_ctas=ctas)
        heap.mark()
        flat = red.allocator(biggest // 4, torch.float32)
        heap.sync_group()
        for mib in args.sizes_mib:
            n = int(mib * (1 << 20)) // 4
            torch.manual_seed(7 + rank)
            vals = torch.randn(n, device=device)
            ref = vals.clone()
            dist.all_reduce(ref)
            ref /= world
            flat[:n].copy_(vals)
            red.reduce(flat[:n], 1.0 / world)
            torch.cuda.synchronize()
            err = (flat[:n] - ref).abs().max().item()
            if err > 1e-5 * (ref.abs().max().item() + 1):
                raise AssertionError(f"two-shot all-reduce differs from the library's by {err}")
            scratch = vals.clone()
            t_nccl = _time(lambda: dist.all_reduce(scratch.mul_(1.0 / world)))
            t_symm = _time(lambda: red.reduce(flat[:n], 1.0 / world))
            bus = lambda ms: 2 * (world - 1) / world * n * 4 / ms / 1e6       # noqa: E731
            common.p0(f"allreduce {mib} MiB fp32, {ctas} CTAs: nccl={t_nccl:.3f}ms({bus(t_nccl):.0f}GB/s bus) "
                      f"symm_two_shot={t_symm:.3f}ms({bus(t_symm):.0f}GB/s bus)")
        heap.release_to_mark()
    gemm_status()


def gemm_status():
    from ..ops import gemm
    gemm.check_status()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mib", type=float, nargs="+", default=[0.5, 2, 8, 32, 128])
    ap.add_argument("--allreduce", action="store_true")
    ap.add_argument("--ctas", type=int, nargs="+", default=[24], help="CTA counts of the two-shot kernel to try")
    ap.add_argument("--iters", type=int, default=_ITERS, help="timed repetitions per size and method")
    ap.add_argument("--warmup", type=int, default=_WARMUP, help="untimed repetitions before them")
    args = ap.parse_args(argv)
    global _ITERS, _WARMUP
    _ITERS, _WARMUP = max(1, args.iters), max(0, args.warmup)
    device = init_distributed()
    rank, world = dist.get_rank(), dist.get_world_size()
    if args.allreduce:
        bench_allreduce(args, device, rank, world)
        dist.barrier()
        dist.destroy_process_group()
        return
    from ..parallel.symm import SymmAllToAll, SymmetricHeap
    heap = SymmetricHeap(None, int(max(args.sizes_mib) * (1 << 20) * world * 2 + (64 << 20)), device)
    partners = partner_table(world)[rank]
    for mib in args.sizes_mib:
        n = int(mib * (1 << 20)) // 4
        send = _pattern(rank, world, n, device)
        recv = torch.empty_like(send)

        def nccl_a2a():
            dist.all_to_all_single(recv, send)

        def nccl_rr():
            recv[rank].copy_(send[rank])
            for q in partners:
                if q < 0:
                    continue
                ops = [dist.P2POp(dist.irecv, recv[q], q), dist.P2POp(dist.isend, send[q], q)]
                for r in dist.batch_isend_irecv(ops):
                    r.wait()

        a2a = SymmAllToAll(heap, n * 4)
        results = {}
        for name, fn in (("nccl_a2a", nccl_a2a), ("nccl_round_robin", nccl_rr)):
            recv.zero_()
            fn()
            torch.cuda.synchronize()
            _check(recv, rank, world, n, device, name)
            results[name] = _time(fn)
        out = a2a(send)
        torch.cuda.synchronize()
        _check(out, rank, world, n, device, "symm_a2a")
        results["symm_a2a"] = _time(lambda: a2a(send))
        per_peer = n * 4
        line = " ".join(f"{k}={v:.3f}ms({per_peer * (world - 1) / v / 1e6:.1f}GB/s)" for k, v in results.items())
        common.p0(f"per-peer {mib} MiB: {line}")
        heap.release_to_mark() if heap._marks else None
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
