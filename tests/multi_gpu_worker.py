"""Worker run under torchrun by the multi-GPU tests (one process per GPU, NCCL).

Checks, in order: bit-exact device-initiated all-to-all against a computed pattern and against
NCCL; the kernel-side barrier; the peer-memory all-reduce against NCCL; the fused MoE exchange
(forward and backward of a whole layer) against the plain all-to-all transport; and that a wait
nobody satisfies returns a status instead of hanging.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from fluidmoe_b200.distributed import init_distributed, init_parallel
    from fluidmoe_b200.ops import gemm
    from fluidmoe_b200.parallel.symm import SymmAllReduce, SymmAllToAll, SymmetricHeap
    from fluidmoe_b200 import _native

    dev = init_distributed()
    rank, world = dist.get_rank(), dist.get_world_size()
    heap = SymmetricHeap(None, 512 << 20, dev)

    # ---- 1. all-to-all: pattern derived from (sender, receiver, index), bit-exact ----
    n = 1 << 18
    a2a = SymmAllToAll(heap, n * 4)
    for it in range(3):
        idx = torch.arange(n, device=dev, dtype=torch.int32)
        send = torch.stack([(rank * 1000003 + p * 7919 + it) + idx for p in range(world)]).contiguous()
        got = a2a(send).clone()
        torch.cuda.synchronize()
        for p in range(world):
            exp = (p * 1000003 + rank * 7919 + it) + idx
            assert torch.equal(got[p], exp), f"a2a mismatch from {p} on {rank} iter {it}"
        ref = torch.empty_like(send)
        dist.all_to_all_single(ref, send)
        assert torch.equal(got, ref)
    heap.barrier()
    torch.cuda.synchronize()
    gemm.check_status()

    # ---- 2. all-reduce over peer memory vs NCCL ----
    for dtype in (torch.float32, torch.bfloat16):
        ar = SymmAllReduce(heap, 1 << 20, dtype)
        for it in range(2):
            torch.manual_seed(100 * it + rank)
            x = torch.randn(1 << 20, device=dev).to(dtype)
            ar.buf.local.copy_(x)
            ref = x.float().clone()
            dist.all_reduce(ref)
            out = ar(scale=1.0 / world).float()
            torch.cuda.synchronize()
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert (out - ref / world).abs().max().item() <= tol * (ref.abs().max().item() / world + 1), dtype
    gemm.check_status()

    # ---- 2b. in-switch (NVLS) all-reduce, where the system offers a multicast mapping ----
    from fluidmoe_b200.parallel.symm import NvlsAllReduce
    nv = NvlsAllReduce(heap, (1 << 20) + 3) if os.environ.get("FLUIDMOE_TEST_NVLS", "0") == "1" else None
    if nv is None:
        pass
    elif nv.available:
        for it in range(2):
            torch.manual_seed(200 * it + rank)
            x = torch.randn((1 << 20) + 3, device=dev)
            nv.local.copy_(x)
            ref = x.clone()
            dist.all_reduce(ref)
            out = nv(scale=1.0 / world)
            torch.cuda.synchronize()
            assert (out - ref / world).abs().max().item() <= 1e-5 * (ref.abs().max().item() / world + 1)
        gemm.check_status()
        if rank == 0:
            print("NVLS_ALLREDUCE_OK", flush=True)
    elif rank == 0:
        print("NVLS_ALLREDUCE_SKIPPED (no multicast mapping)", flush=True)

    # ---- 3. a wait that nothing satisfies returns a status (bounded wait) ----
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    st = gemm.status_buffer(dev)
    _native.lib().wait_flag(flag.data_ptr(), 1, int(50e6), st.data_ptr(), _native.stream_ptr())
    torch.cuda.synchronize()
    try:
        gemm.check_status()
        raise AssertionError("expected a timeout status")
    except gemm.FluidKernelTimeout:
        pass
    # the context is still usable
    assert torch.ones(4, device=dev).sum().item() == 4.0
    heap.close()

    # ---- 4. fused MoE exchange inside a whole layer vs the all-to-all transport ----
    from fluidmoe_b200.models.transformer import TransformerLayer
    from fluidmoe_b200.ops.rope import make_rope_freqs
    from fluidmoe_b200.parallel.scheduler import get_backward_scheduler

    pc = init_parallel(ep_size=world, device=dev, symmetric_heap_bytes=1 << 30)
    sched = get_backward_scheduler()
    H, nh, nkv, F, E, k = 1024, 8, 8, 1024, 8, 8     # k == E: no discrete routing flips
    s_loc, b = 512, 1
    kw = dict(dtype=torch.bfloat16, device=dev, router_dtype=torch.float32, activation_func="swiglu",
              norm_type="rmsnorm", init_std=0.05)
    results = {}
    for mode in ("a2a", "p2p", "fused"):
        torch.manual_seed(7)
        layer = TransformerLayer(H, nh, nkv, F, E, k, pc.cp_group, pc.ep_group, comm_mode=mode,
                                 parallel_ctx=pc if mode == "fused" else None, **kw)
        # same dense weights everywhere; expert weights differ per rank by construction order,
        # so seed them per rank explicitly
        with torch.no_grad():
            g = torch.Generator(device=dev).manual_seed(1000 + rank)
            layer.moe_w1.copy_((torch.randn(layer.moe_w1.shape, device=dev, generator=g) * 0.05).bfloat16())
            layer.moe_w2.copy_((torch.randn(layer.moe_w2.shape, device=dev, generator=g) * 0.05).bfloat16())
        sched.disable()
        torch.manual_seed(11 + rank)
        x = torch.randn(s_loc, b, H, device=dev).bfloat16().requires_grad_(True)
        gy = torch.randn(s_loc, b, H, device=dev).bfloat16()
        rot = make_rope_freqs(s_loc * world, 64, device=dev)
        for it in range(2):       # twice: buffers and counters must be reusable
            x.grad = None
            for p_ in layer.parameters():
                p_.grad = None
            y = layer(x, rot)
            y.backward(gy)
            if mode == "fused":
                pc.fused_ctx.iteration_barrier()
        torch.cuda.synchronize()
        gemm.check_status()
        results[mode] = (y.detach().float(), x.grad.float(), {n_: p_.grad.float() for n_, p_ in layer.named_parameters()})

    def fro(a, b_):
        return ((a - b_).norm() / (b_.norm() + 1e-9)).item()
    yb, gxb, gb = results["a2a"]
    for mode in ("p2p", "fused"):
        y, gx, g = results[mode]
        assert fro(y, yb) < 2e-2, (mode, "y", fro(y, yb))
        assert fro(gx, gxb) < 3e-2, (mode, "dx", fro(gx, gxb))
        for n_ in gb:
            assert fro(g[n_], gb[n_]) < 3e-2, (mode, n_, fro(g[n_], gb[n_]))
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK", world, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
