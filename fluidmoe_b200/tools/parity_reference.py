"""Numerical parity with the reference implementation on an identical architecture.

    python -m fluidmoe_b200.tools.parity_reference --ref-root baseline/_ref
    torchrun --nproc-per-node N -m fluidmoe_b200.tools.parity_reference --ref-root baseline/_ref

Builds the reference's ``fluid.layer.transformer.TransformerModel`` (GELU experts, LayerNorm with
bias, padded capacity 1.0: the only architecture it has) from an installed copy of the reference,
loads its ``state_dict`` into this framework's ``TransformerModel`` through
``load_reference_state_dict`` and runs both on the same inputs with sequence / expert parallelism
over all ranks:

1. one forward + backward: output, input gradient and every parameter gradient are compared
   (relative Frobenius error; reduced gradients are read from ``param.main_grad`` of both);
2. a short training run of both stacks inside the same torch harness (embedding, final LayerNorm,
   head, cross-entropy, ``torch.optim.AdamW``), same data, same initial weights: the two loss
   curves are printed side by side, which is how the reference validates itself end to end
   (examples/run_training.sh:243-290 prints final loss and gradient norm of each arm; its layer
   matches Megatron's initialisation for the same purpose, fluid/layer/transformer.py:981-1056).

Rank 0 prints ``PARITY ...`` lines and one final ``PARITY_RESULT {json}``; the exit code is 0 when
every bound holds.  Needs CUDA (the reference has no CPU path).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F


def _fro(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _import_reference(ref_root: str):
    ref_root = os.path.abspath(ref_root)
    if not os.path.isdir(os.path.join(ref_root, "fluid")):
        raise SystemExit(f"no reference package under {ref_root}")
    sys.path.insert(0, ref_root)
    for k in [k for k in sys.modules if k == "fluid" or k.startswith("fluid.")]:
        del sys.modules[k]
    import fluid  # noqa: F401 - the reference package, not this repository's alias package
    assert os.path.abspath(fluid.__file__).startswith(ref_root), fluid.__file__
    from fluid.core.scheduler import get_backward_scheduler as ref_sched
    import fluid.layer.transformer as ref_mod
    return ref_mod.TransformerModel, ref_sched, ref_mod


class _Arm:
    """One decoder stack inside a common torch harness (embedding, final norm, head, loss, AdamW)."""

    def __init__(self, name, decoder, sched, vocab, hidden, device, rotary, world, finish, begin, lr):
        self.name, self.decoder, self.sched, self.world = name, decoder, sched, world
        self.rotary, self.finish, self.begin = rotary, finish, begin
        g = torch.Generator(device=device).manual_seed(4321)
        self.emb = torch.nn.Embedding(vocab, hidden, dtype=torch.bfloat16, device=device)
        self.norm = torch.nn.LayerNorm(hidden, dtype=torch.bfloat16, device=device)
        self.head = torch.nn.Linear(hidden, vocab, bias=False, dtype=torch.bfloat16, device=device)
        with torch.no_grad():
            self.emb.weight.copy_(torch.randn(vocab, hidden, device=device, generator=g) * 0.02)
            self.head.weight.copy_(torch.randn(vocab, hidden, device=device, generator=g) * 0.02)
        self.extra = list(self.emb.parameters()) + list(self.norm.parameters()) + list(self.head.parameters())
        self.params = list(decoder.parameters()) + self.extra
        self.opt = torch.optim.AdamW(self.params, lr=lr, weight_decay=0.0)

    def step(self, ids_full):
        for p in self.params:
            p.grad = None
            if hasattr(p, "_ar_buf_written"):
                p._ar_buf_written = False
        self.begin()
        ids, labels = ids_full[:-1], ids_full[1:]
        x = self.emb(ids)
        for layer in self.decoder.layers:
            x = layer(x, self.rotary)
        logits = self.head(self.norm(x))
        loss = F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.reshape(-1))
        loss.backward()
        self.finish()
        if self.world > 1:
            for p in self.extra:
                p.grad.div_(self.world)
                dist.all_reduce(p.grad)
        sq = torch.zeros((), device=loss.device)
        for p in self.decoder.parameters():
            mg = getattr(p, "main_grad", None)
            if mg is not None and getattr(p, "_ar_buf_written", True):
                p.grad = mg if mg.dtype == p.dtype else mg.to(p.dtype)
            if p.grad is not None:
                sq += p.grad.float().pow(2).sum()
        self.opt.step()
        self.sched.clear_iteration()
        lv = loss.detach().float().clone()
        if self.world > 1:
            dist.all_reduce(lv)
            lv /= self.world
        return lv.item(), sq.sqrt().item()


def _diagnose(ref, ours, x0, rotary, say, world) -> None:
    """Black-box split of the first layer: with ``moe_w2 = 0`` the layer returns ``x + attention``,
    with ``proj_weight = 0`` it returns ``x + MoE(norm2(x))``."""
    lr, lo = ref.layers[0], ours.layers[0]

    def delta(layer, rot):
        with torch.no_grad():
            return (layer(x0, rot) - x0).float()

    def both(tag, rot):
        dr, do = delta(lr, rot), delta(lo, rot)
        e = torch.tensor([(do - dr).norm().item() ** 2, dr.norm().item() ** 2, do.norm().item() ** 2],
                         device=x0.device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(e)
        e = e.sqrt().tolist()
        say(f"PARITY diagnose {tag:34s} |ours - ref| {e[0]:.4e}  |ref| {e[1]:.4e}  |ours| {e[2]:.4e}  "
            f"rel {e[0] / (e[1] + 1e-12):.3e}")

    both("layer 0, full, rotary", rotary)
    saved = {}
    for name in ("moe_w2", "proj_weight"):
        saved[name] = (getattr(lr, name).detach().clone(), getattr(lo, name).detach().clone())
    with torch.no_grad():
        lr.moe_w2.zero_(); lo.moe_w2.zero_()
    both("attention half, rotary", rotary)
    both("attention half, no rotary", None)
    with torch.no_grad():
        lr.moe_w2.copy_(saved["moe_w2"][0]); lo.moe_w2.copy_(saved["moe_w2"][1])
        lr.proj_weight.zero_(); lo.proj_weight.zero_()
    both("MoE half", rotary)
    with torch.no_grad():
        lr.proj_weight.copy_(saved["proj_weight"][0]); lo.proj_weight.copy_(saved["proj_weight"][1])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default=os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__)))), "baseline", "_ref"))
    ap.add_argument("--layers", type=int, default=2)
    # grouped-query heads: with one query head per KV head the reference's q is a view of a receive
    # buffer that all its layers share, and its saved attention graph breaks from the second layer on
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=8192)
    ap.add_argument("--seq", type=int, default=1024, help="positions per rank")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--chunks", type=int, default=2)
    ap.add_argument("--ref-attn-chunks", type=int, default=1,
                    help="chunk count of the reference's two attention regions.  Both of its chunked paths "
                         "misplace sequence rows on more than one rank: attn_proj writes the all-to-all output of "
                         "chunk c at rows [c*P*sc, (c+1)*P*sc), i.e. in (chunk, rank, row) order instead of the "
                         "(rank, chunk, row) order of the full sequence (fluid/attention/backward.py:131-162), and "
                         "attn_qkv slices the FULL sequence and lets the all-to-all split every slice over the ranks "
                         "(fluid/attention/backward.py:330-349).  1 keeps the reference on its correct paths; any "
                         "other value reproduces its wrong attention gradients")
    ap.add_argument("--comm", default="auto", choices=["auto", "a2a", "p2p", "fused"])
    ap.add_argument("--tol-out", type=float, default=2e-2)
    ap.add_argument("--tol-grad", type=float, default=5e-2)
    ap.add_argument("--tol-loss", type=float, default=1e-2)
    ap.add_argument("--own-routing", action="store_true",
                    help="let this framework's router pick experts itself in the one-step comparison; by default "
                         "the reference's top-k selection is replayed (force_routing), which removes the few tokens "
                         "whose near-tied logits the two bf16 pipelines order differently")
    ap.add_argument("--diagnose", action="store_true",
                    help="also compare the first layer's attention half and MoE half in isolation (by zeroing "
                         "the other half's output weights in both models) and print the norms of the differences")
    args = ap.parse_args(argv)

    os.environ.setdefault("FLUIDMOE_P2P_BACKEND", "nccl")
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "1")
    RefModel, ref_sched_fn, ref_mod = _import_reference(args.ref_root)
    from ..distributed import init_parallel
    from ..models.transformer import TransformerModel
    from ..ops import gemm
    from ..parallel.scheduler import get_backward_scheduler
    from ..utils.checkpoint import load_reference_state_dict

    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    all_group = dist.new_group(list(range(world)))
    ref_group = dist.new_group(list(range(world)))
    pc = init_parallel(ep_size=world, device=device,
                       symmetric_heap_bytes=(2 << 30) if (world > 1 and args.comm in ("auto", "fused")) else 0)
    say = (lambda *a: print(*a, flush=True)) if rank == 0 else (lambda *a: None)
    if world == 1:
        say("PARITY note: with one rank the reference skips its local expert FFN (its local FC1 call is inside "
            "the per-partner loop, fluid/moe/forward.py:690-728) and returns stale buffer contents for the MoE "
            "half; the comparison below is only meaningful from two ranks up")
    H, s_loc, b = args.hidden, args.seq, 1
    d = H // args.heads
    chunk_kw = dict(moe_combine_chunks=args.chunks, moe_dispatch_chunks=args.chunks,
                    attn_proj_chunks=args.chunks, attn_qkv_chunks=args.chunks)

    # ---- the two decoders, identical weights ----
    torch.manual_seed(1234)
    ref = RefModel(num_layers=args.layers, hidden_size=H, num_heads=args.heads, num_kv_heads=args.kv_heads,
                   ffn_hidden_size=args.ffn, num_experts=args.experts, top_k=args.top_k, cp_group=ref_group,
                   ep_group=ref_group, capacity_factor=1.0, dtype=torch.bfloat16, device=device,
                   router_dtype=torch.float32, **{**chunk_kw, "attn_qkv_chunks": args.ref_attn_chunks, "attn_proj_chunks": args.ref_attn_chunks})
    ours = TransformerModel(args.layers, H, args.heads, args.kv_heads, args.ffn, args.experts, args.top_k,
                            pc.cp_group, pc.ep_group, activation_func="gelu", capacity_factor=1.0,
                            dtype=torch.bfloat16, device=device, router_dtype=torch.float32,
                            norm_type="layernorm", comm_mode=args.comm, parallel_ctx=pc, **chunk_kw)
    missing = load_reference_state_dict(ours, ref.state_dict(), strict=True)
    say(f"PARITY state_dict loaded: {len(ref.state_dict())} tensors, missing={list(missing.missing_keys)} "
        f"unexpected={list(missing.unexpected_keys)}")
    ref.prepare_chunk_status(torch.empty(s_loc, b, H, dtype=torch.bfloat16, device=device))
    rs, os_ = ref_sched_fn(), get_backward_scheduler()
    gaps = {"moe_combine": 0.5, "moe_dispatch": 0.5, "attn_proj": 0.3, "attn_qkv": 0.3}
    rs.enable()
    rs.configure_allreduce(enabled=True, shared_dp_group=all_group, expert_dp_group=None, gap_budgets=gaps,
                           shared_ar_bw=3.0e8, expert_ar_bw=3.0e8)
    ref.setup_ar_buffer()
    os_.enable(device)
    os_.configure_allreduce(True, pc.dp_cp_group, pc.expert_dp_group, gaps, 3.0e8, 3.0e8)
    os_.eager_ar = pc.fused_ctx is not None
    ours.setup_ar_buffer()

    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32, device=device) / d))
    fr = torch.outer(torch.arange(s_loc * world, dtype=torch.float32, device=device), inv)
    rotary = torch.cat([fr, fr], dim=-1).view(s_loc * world, 1, 1, d)

    def ours_begin():
        os_.shared_buffer.reset_cursors()
        os_.expert_buffer.reset_cursors()

    def ours_finish():
        os_.finish_batch()
        if pc.fused_ctx is not None:
            pc.fused_ctx.iteration_barrier()

    # ---- 1. one forward + backward on the same activations ----
    g = torch.Generator(device=device).manual_seed(77 + rank)
    x0 = torch.randn(s_loc, b, H, device=device, generator=g).bfloat16()
    dy = (torch.randn(s_loc, b, H, device=device, generator=g) / (s_loc * world)).bfloat16()
    res = {}
    # record the reference's expert selection (one call of its router per layer) to replay it
    picked = []
    ref_router = ref_mod.router_forward

    def recording_router(*a, **kw):
        out = ref_router(*a, **kw)
        picked.append(out[4].detach().clone())        # top_indices [tokens, k]
        return out
    for name, model, begin, finish, sched in (("reference", ref, lambda: None, rs.finish_batch, rs),
                                              ("ours", ours, ours_begin, ours_finish, os_)):
        if name == "reference":
            ref_mod.router_forward = recording_router
        elif not args.own_routing:
            for layer, idx in zip(model.layers, picked):
                layer.force_routing(idx)
        for p in model.parameters():
            p.grad = None
            if hasattr(p, "_ar_buf_written"):
                p._ar_buf_written = False
        begin()
        x = x0.clone().requires_grad_(True)
        y = x
        for layer in model.layers:
            y = layer(y, rotary)
        y.backward(dy)
        finish()
        torch.cuda.synchronize()
        grads = {n: (p.main_grad if getattr(p, "main_grad", None) is not None else p.grad).float().clone()
                 for n, p in model.named_parameters()}
        res[name] = (y.detach().float(), x.grad.float(), grads)
        sched.clear_iteration()
        if name == "reference":
            ref_mod.router_forward = ref_router
        else:
            for layer in model.layers:
                layer.force_routing(None)
    gemm.check_status()
    yr, dxr, gr = res["reference"]
    yo, dxo, go = res["ours"]
    errs = {"y": _fro(yo, yr), "dx": _fro(dxo, dxr)}
    for n in gr:
        errs["grad:" + n] = _fro(go[n], gr[n])
    if args.diagnose:
        for n in gr:
            a_, b_ = go[n].flatten(), gr[n].flatten()
            cos = torch.dot(a_, b_) / (a_.norm() * b_.norm() + 1e-30)
            print(f"PARITY rank {rank} {n:28s} err {errs['grad:' + n]:.3e}  |ours|/|ref| "
                  f"{(a_.norm() / (b_.norm() + 1e-30)).item():.4f}  cosine {cos.item():.4f}", flush=True)
    t = torch.tensor(list(errs.values()), device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    errs = dict(zip(errs.keys(), t.tolist()))
    worst_grad = max(v for k_, v in errs.items() if k_ != "y")
    say(f"PARITY world={world} step0: y {errs['y']:.3e}  dx {errs['dx']:.3e}  worst gradient {worst_grad:.3e}")
    for k_, v in errs.items():
        if k_.startswith("grad:"):
            say(f"PARITY   {k_[5:]:28s} {v:.3e}")

    if args.diagnose:
        _diagnose(ref, ours, x0, rotary, say, world)

    # ---- 2. short training run of both stacks in the same harness ----
    arms = [
        _Arm("reference", ref, rs, args.vocab, H, device, rotary, world, rs.finish_batch, lambda: None, args.lr),
        _Arm("ours", ours, os_, args.vocab, H, device, rotary, world, ours_finish, ours_begin, args.lr),
    ]
    gh = torch.Generator().manual_seed(100 + rank)
    batches = [torch.randint(0, args.vocab, (s_loc + 1, b), generator=gh).to(device) for _ in range(4)]
    curves = {a.name: [] for a in arms}
    norms = {a.name: [] for a in arms}
    for i in range(max(args.steps, 1)):
        for a in arms:
            lv, gn = a.step(batches[i % len(batches)])
            curves[a.name].append(lv)
            norms[a.name].append(gn)
    torch.cuda.synchronize()
    gemm.check_status()
    say("PARITY step   loss(reference)  loss(ours)   |grad|(reference)  |grad|(ours)")
    for i in range(args.steps):
        say(f"PARITY {i:4d}   {curves['reference'][i]:14.5f}  {curves['ours'][i]:10.5f}   "
            f"{norms['reference'][i]:14.5f}  {norms['ours'][i]:10.5f}")
    loss0 = abs(curves["ours"][0] - curves["reference"][0]) / abs(curves["reference"][0])
    drift = max(abs(o - r) / abs(r) for o, r in zip(curves["ours"], curves["reference"]))
    ok = errs["y"] < args.tol_out and worst_grad < args.tol_grad and loss0 < args.tol_loss
    say("PARITY_RESULT " + json.dumps({
        "world": world, "comm": args.comm if world > 1 else "local", "y_err": errs["y"], "dx_err": errs["dx"],
        "worst_grad_err": worst_grad, "loss_step0_rel": loss0, "loss_curve_max_rel": drift,
        "loss_reference": curves["reference"], "loss_ours": curves["ours"], "ok": bool(ok)}))
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
