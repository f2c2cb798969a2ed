#!/usr/bin/env python
"""Flagship benchmark: training step of a 4-layer Mixtral-shaped MoE transformer.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...        # the unmodified reference from baseline/_ref

Model: hidden 4096, 32 query / 8 KV heads (d = 128), causal, RoPE, 8 experts top-2 with FFN
14336, vocabulary 32000, 4096 positions per rank (weak scaling: SP = EP = N), batch 1,
cross-entropy on shifted ids, backward scheduler on with 4 dX chunks, optimizer step included.
The arm of this repository uses SwiGLU experts and RMSNorm; the reference has neither, so its arm
runs GELU experts with FFN 21504 (the same FLOPs and weight bytes as SwiGLU 14336) and LayerNorm.

Prints one JSON line on rank 0 (see the keys at the bottom of ``main``).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))

MODEL = dict(hidden=4096, heads=32, kv_heads=8, ffn=14336, experts=8, top_k=2, vocab=32000, layers=4,
             seq_per_rank=4096, batch=1)
BASELINE_TOKENS_PER_S = None  # the reference publishes no tokens/s figure for this configuration
METRIC_TRAIN = "MoE transformer training tokens/s (fwd+bwd+optimizer, 4-layer Mixtral-shaped block stack)"
METRIC_FWD = "MoE transformer forward (inference) tokens/s (4-layer Mixtral-shaped block stack, loss included)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL["layers"])
    ap.add_argument("--seq", type=int, default=MODEL["seq_per_rank"])
    ap.add_argument("--chunks", type=int, default=4)
    ap.add_argument("--mode", default="full", choices=["F", "FB", "full"])
    ap.add_argument("--comm", default="auto", choices=["auto", "a2a", "p2p", "fused"])
    ap.add_argument("--tiny", action="store_true", help="small shapes for a functional check")
    ap.add_argument("--opt-state", default="bf16", choices=["bf16", "fp32"],
                    help="dtype of the Adam moments (torch.optim.AdamW keeps bf16 moments for bf16 parameters)")
    ap.add_argument("--fuse-optimizer", type=int, default=1,
                    help="Adam for the expert weights inside the backward pass (bf16 moments, scheduler on, one "
                         "micro-batch per step): 1 = in the weight-gradient GEMM epilogue, 2 = small-CTA kernel on "
                         "a side stream behind each weight-gradient GEMM, 0 = off")
    ap.add_argument("--profile", default="", help="write a torch-profiler kernel table of one step to this file")
    ap.add_argument("--arch", default="native", choices=["native", "matched"],
                    help="native: SwiGLU 14336 + RMSNorm (this repository's arm of the headline); matched: the "
                         "reference's own architecture (GELU ffn 21504, LayerNorm, padded capacity 1.0) so that "
                         "both arms run the identical model")
    ap.add_argument("--forward-only", action="store_true",
                    help="time the forward pass alone (inference latency): no backward, no optimizer")
    ap.add_argument("--dw-side-ctas", type=int, default=0,
                    help="> 0: deferred weight-gradient GEMMs run on a low-priority side stream with at most this "
                         "many CTAs, concurrently with the critical path (0: on the compute stream, the default)")
    ap.add_argument("--grad-reduce", default="", choices=["", "nccl", "symm"],
                    help="dense-gradient all-reduce: library (nccl) or this repository's two-shot kernel over peer "
                         "memory (symm); default: FLUIDMOE_GRAD_REDUCE or nccl")
    ap.add_argument("--recompute-fc1", action="store_true",
                    help="do not keep the FC1 pre-activation; rebuild it in the backward pass (saves memory, costs one GEMM)")
    ap.add_argument("--loss-trace", action="store_true", help="add the loss of every timed end-to-end step to the JSON line")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------
# helpers shared by both arms
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        busy = [c for c, p in zip(sm, power) if p > 300] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def timed_region(torch, dist, world, fn_step, steps):
    """Barrier + synchronize on both sides; device time by CUDA events; max over ranks."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    s.record()
    for i in range(steps):
        fn_step(i)
    e.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e3
    if world > 1:
        dist.barrier()
    ms = s.elapsed_time(e)
    t = torch.tensor([ms, wall], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t[0].item(), t[1].item()


class LossReader:
    """Device-to-host read of every step's loss without stalling the launch queue: the 4-byte value is
    copied into a pinned buffer right behind the step and read on the host one step later (the last
    one at the end of the timed loop), the way a training loop logs its loss."""

    def __init__(self, torch, steps):
        self.torch, self.steps = torch, steps
        self.buf = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(2)]
        self.ev = [torch.cuda.Event() for _ in range(2)]
        self.pending = None
        self.values = []

    def _consume(self):
        if self.pending is not None:
            self.ev[self.pending].synchronize()
            self.values.append(float(self.buf[self.pending]))
            self.pending = None

    def submit(self, i, loss):
        slot = i & 1
        self._consume()                       # the previous step's value: its copy finished long ago
        self.buf[slot].copy_(loss.detach().float(), non_blocking=True)
        self.ev[slot].record()
        self.pending = slot
        if i == self.steps - 1:
            self._consume()                   # the last step is read before the timed loop ends


def make_batches(torch, n, seq, batch, vocab, seed):
    """Pinned host batches of token ids, one extra position for the shifted labels."""
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (seq + 1, batch), generator=g).pin_memory() for _ in range(n)]


def emit(rank, payload):
    if rank == 0:
        print(json.dumps(payload), flush=True)


# ------------------------------------------------------------------------------------------------
# this repository's arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    from fluidmoe_b200.distributed import init_distributed, init_parallel
    from fluidmoe_b200.models.gpt import MoEGPT
    from fluidmoe_b200.ops import elementwise, gemm
    from fluidmoe_b200.ops.optim import FusedAdam
    from fluidmoe_b200.parallel.ddp import FluidDDP, FluidOptimizerWrapper
    from fluidmoe_b200.parallel.scheduler import get_backward_scheduler

    rank, local_rank, world = dist_env()
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")
    device = init_distributed()
    m = dict(MODEL)
    if args.tiny:
        m.update(hidden=512, heads=8, kv_heads=8, ffn=1024, vocab=2048)
        args.seq = min(args.seq, 512)
    heap = (6 << 30) if (world > 1 and args.comm in ("auto", "fused")) else 0
    if heap and (args.grad_reduce or os.environ.get("FLUIDMOE_GRAD_REDUCE", "")) == "symm":
        heap += 2 << 30        # the dense flat gradient buffer moves into the symmetric heap
    pc = init_parallel(ep_size=world, device=device, symmetric_heap_bytes=heap)
    torch.manual_seed(1234)
    matched = args.arch == "matched"
    ffn = m["ffn"] * 3 // 2 if matched else m["ffn"]
    act_name, norm_name = ("gelu", "layernorm") if matched else ("swiglu", "rmsnorm")
    model = MoEGPT(m["vocab"], args.layers, m["hidden"], m["heads"], m["kv_heads"], ffn, m["experts"],
                   m["top_k"], pc.cp_group, pc.ep_group, dtype=torch.bfloat16, device=device,
                   router_dtype=torch.float32, activation_func=act_name, norm_type=norm_name,
                   moe_combine_chunks=args.chunks, moe_dispatch_chunks=args.chunks,
                   attn_proj_chunks=args.chunks, attn_qkv_chunks=args.chunks, comm_mode=args.comm,
                   parallel_ctx=pc, recompute_fc1=args.recompute_fc1)
    sched = get_backward_scheduler()
    if args.mode == "F":
        sched.disable()
    else:
        sched.enable(device)
    # knobs the tuner measured on this kind of box (tools/tune.py writes tools/tuned_defaults.json);
    # a flag given on the command line wins
    from fluidmoe_b200.tools.experiment_configs import get_block_benchmark_defaults
    tuned_fused = get_block_benchmark_defaults(os.environ.get("FLUIDMOE_TUNED_NODE", "b200_2gpu_fused"))
    tuned_p2p = get_block_benchmark_defaults(os.environ.get("FLUIDMOE_TUNED_NODE_P2P", "b200_2gpu_p2p"))
    ar_bw = float(tuned_p2p.get("shared_ar_bw") or 3.0e8)
    grad_reduce = args.grad_reduce or (tuned_fused.get("fused_grad_reduce") if heap else None) or None
    ddp = FluidDDP(None, model, sched, dp_cp_group=pc.dp_cp_group, expert_dp_group=pc.expert_dp_group,
                   ar_enabled=args.mode == "full",
                   gap_budgets={"moe_combine": 0.5, "moe_dispatch": 0.5, "attn_proj": 0.3, "attn_qkv": 0.3},
                   shared_ar_bw=ar_bw, expert_ar_bw=ar_bw, grad_reduce=grad_reduce)
    sched.eager_ar_min_bytes = int(tuned_fused.get("fused_eager_ar_min_bytes", sched.eager_ar_min_bytes))
    if args.dw_side_ctas == 0:
        args.dw_side_ctas = int(tuned_fused.get("fused_dw_side_ctas", 0))
    opt = FluidOptimizerWrapper(
        FusedAdam(model.parameters(), lr=1e-4, weight_decay=0.0,
                  state_dtype=torch.bfloat16 if args.opt_state == "bf16" else torch.float32), sched)
    if args.dw_side_ctas > 0:
        sched.dw_on_side_stream, sched.dw_max_ctas = True, args.dw_side_ctas
    fused_params = 0
    if args.fuse_optimizer and args.mode != "F" and args.opt_state == "bf16":
        fused_params = opt.fuse_into_backward(mode="stream" if args.fuse_optimizer == 2 else "epilogue")
    seq, batch = args.seq, m["batch"]
    n_batches = 4
    host = make_batches(torch, n_batches, seq, batch, m["vocab"], 100 + rank)
    dev_batches = [b.to(device) for b in host]
    last = {}

    trace = []

    def train_step(ids_full):
        if args.forward_only:
            with torch.no_grad():
                return ddp(ids_full[:-1], ids_full[1:])
        ddp.zero_grad_buffer()
        loss = ddp(ids_full[:-1], ids_full[1:])
        loss.backward()
        ddp.finish_grad_sync()
        opt.step()
        return loss

    def step_device(i):
        last["loss"] = train_step(dev_batches[i % n_batches])

    reader = LossReader(torch, args.steps)

    def step_e2e(i):
        ids = host[i % n_batches].to(device, non_blocking=True)
        reader.submit(i, train_step(ids))

    for i in range(args.warmup):
        step_device(i)
        if i == 0:
            # a bounded device-side wait that ran out shows up here, before more steps are spent
            torch.cuda.synchronize()
            gemm.check_status()
    torch.cuda.synchronize()
    gemm.check_status()
    if args.profile:
        _profile_one_step(torch, step_device, args.profile, rank)
    l0 = gemm.LAUNCHES + elementwise.LAUNCHES + _extra_launches()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, _ = timed_region(torch, dist, world, step_device, args.steps)
    launches = gemm.LAUNCHES + elementwise.LAUNCHES + _extra_launches() - l0
    _, wall_e2e = timed_region(torch, dist, world, step_e2e, args.steps)
    assert len(reader.values) == args.steps, "every step's loss is read on the host inside the timed region"
    last["loss_val"] = reader.values[-1]
    trace.extend(reader.values)
    clocks = sampler.stop() if rank == 0 else {}
    gemm.check_status()
    tokens = world * seq * batch * args.steps
    value = tokens / (ms / 1e3)
    e2e = tokens / (wall_e2e / 1e3)
    emit(rank, {
        "metric": METRIC_FWD if args.forward_only else METRIC_TRAIN,
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)", "impl": "ours",
        "config": {"model": "mixtral-8x7b-shaped, %d layers, hidden %d, %d/%d heads, 8 experts top-2 %s ffn %d, %s, vocab %d"
                            % (args.layers, m["hidden"], m["heads"], m["kv_heads"],
                               "GELU" if matched else "SwiGLU", ffn, "LayerNorm" if matched else "RMSNorm", m["vocab"]),
                   "arch": args.arch, "forward_only": bool(args.forward_only),
                   "global_batch": batch, "seq_len": seq * world, "seq_per_rank": seq,
                   "parallelism": f"sp{world}ep{world}", "scheduler_mode": args.mode, "dx_chunks": args.chunks,
                   "comm": args.comm, "adam_moments": args.opt_state, "grad_accum": "fp32",
                   "grad_reduce": ddp.grad_reduce_mode, "dw_side_stream_ctas": args.dw_side_ctas,
                   "recompute_fc1": bool(args.recompute_fc1),
                   "optimizer": ("AdamW every step inside the timed region; expert weights (%d tensors) updated in their "
                                 "weight-gradient GEMM %s, all other parameters by the fused Adam kernel in step()"
                                 % (fused_params, "epilogue" if args.fuse_optimizer != 2 else "stream")) if fused_params
                   else "AdamW (fused kernel) every step inside the timed region", "l2": "working set of a step is several GB (>> 126 MB L2); no explicit flush",
                   "loss": float(last["loss_val"]), **({"loss_trace": trace} if args.loss_trace else {})},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": wall_e2e / args.steps,
                "h2d_bytes_per_step": (seq + 1) * batch * 8, "d2h_bytes_per_step": 4,
                "loss_readback": "copied to pinned memory behind every step, read on the host one step later (last step at the end of the loop)"},
        "gpu_launches": int(launches),
    })
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _profile_one_step(torch, step_fn, path, rank=0):
    """Every rank runs the step (its kernels wait for the peers'); only rank 0 records it."""
    from torch.profiler import ProfilerActivity, profile
    if rank != 0:
        step_fn(0)
        torch.cuda.synchronize()
        return
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        step_fn(0)
        torch.cuda.synchronize()
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=45, max_name_column_width=90))
        # where the device sat idle: the largest gaps between consecutive kernels on the timeline
        from fluidmoe_b200.utils.timeline import idle_gaps, merge_intervals, overlap
        evs = []
        for ev in prof.events():
            tr = getattr(ev, "time_range", None)
            if ev.device_time_total > 0 and tr is not None and str(getattr(ev, "device_type", "")).endswith("CUDA"):
                evs.append((tr.start, tr.end, ev.name))
        span, idle, gaps = idle_gaps(evs)
        if evs:
            f.write("\n\ndevice timeline: %.3f ms from first kernel start to last kernel end, %.3f ms idle in %d gaps; "
                    "largest gaps (us, after -> before):\n" % (span / 1e3, idle / 1e3, len(gaps)))
            for g, a, b in sorted(gaps, reverse=True)[:25]:
                f.write(f"{g:10.1f}  {a[:70]}  ->  {b[:70]}\n")
        # a collective that runs beside a persistent GEMM takes SMs from it: show the overlap per launch
        # (the profiler lists a collective twice, as a kernel and as an annotation: the union counts once)
        coll = merge_intervals((st, en) for st, en, name in evs if "nccl" in name.lower() or "allreduce" in name.lower())
        f.write("\n\nper-launch device time of the GEMM kernels (us) and the part of it during which a "
                "collective kernel ran on another stream, in launch order:\n")
        for ev in prof.events():
            if "gemm" in ev.name and "sm100_kernel" in ev.name and ev.device_time_total > 0:
                tr = getattr(ev, "time_range", None)
                ov = overlap(tr.start, tr.end, coll) if tr is not None else 0.0
                f.write(f"{ev.device_time_total:10.1f} {ov:9.1f}  {ev.name[:110]}\n")


def _extra_launches() -> int:
    total = 0
    for name in ("fluidmoe_b200.ops.flash", "fluidmoe_b200.parallel.fused"):
        mod = sys.modules.get(name)
        total += getattr(mod, "LAUNCHES", 0) if mod is not None else 0
    return total


# ------------------------------------------------------------------------------------------------
# reference arm: the unmodified reference package installed under baseline/_ref
# ------------------------------------------------------------------------------------------------
def run_reference(args):
    ref_root = os.path.join(REPO, "baseline", "_ref")
    rank, local_rank, world = dist_env()
    if not os.path.isdir(os.path.join(ref_root, "fluid")):
        emit(0, {"impl": "reference", "unavailable": "baseline/_ref is empty: the reference has no setup.py / "
                 "pyproject.toml; install it from a copy with a packaging shim (pip --no-index --target baseline/_ref)"})
        return
    sys.path.insert(0, ref_root)
    for k in [k for k in sys.modules if k == "fluid" or k.startswith("fluid.")]:
        del sys.modules[k]
    os.environ.setdefault("FLUIDMOE_P2P_BACKEND", "nccl")
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "1")
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    try:
        import fluid  # noqa: F401 - the reference package
        from fluid.core.scheduler import get_backward_scheduler
        from fluid.layer.transformer import TransformerModel
    except Exception as e:  # noqa: BLE001
        emit(rank, {"impl": "reference", "unavailable": f"reference import failed: {type(e).__name__}: {e}"[:300]})
        return
    assert "baseline/_ref" in fluid.__file__.replace(os.sep, "/"), fluid.__file__
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    m = dict(MODEL)
    if args.tiny:
        m.update(hidden=512, heads=8, kv_heads=8, ffn=1024, vocab=2048)
        args.seq = min(args.seq, 512)
    ffn_ref = m["ffn"] * 3 // 2          # GELU (2 matrices) FLOP- and byte-matched to SwiGLU (3 matrices)
    all_group = dist.new_group(list(range(world)))
    cp_group = ep_group = dist.new_group(list(range(world)))
    torch.manual_seed(1234)
    model = TransformerModel(
        num_layers=args.layers, hidden_size=m["hidden"], num_heads=m["heads"], num_kv_heads=m["kv_heads"],
        ffn_hidden_size=ffn_ref, num_experts=m["experts"], top_k=m["top_k"], cp_group=cp_group,
        ep_group=ep_group, moe_combine_chunks=args.chunks, moe_dispatch_chunks=args.chunks,
        attn_proj_chunks=args.chunks, attn_qkv_chunks=args.chunks, capacity_factor=1.0,
        dtype=torch.bfloat16, device=device, router_dtype=torch.float32)
    emb = torch.nn.Embedding(m["vocab"], m["hidden"], dtype=torch.bfloat16, device=device)
    final_norm = torch.nn.LayerNorm(m["hidden"], dtype=torch.bfloat16, device=device)
    head = torch.nn.Linear(m["hidden"], m["vocab"], bias=False, dtype=torch.bfloat16, device=device)
    seq, batch = args.seq, m["batch"]
    x_probe = torch.empty(seq, batch, m["hidden"], dtype=torch.bfloat16, device=device)
    model.prepare_chunk_status(x_probe)
    sched = get_backward_scheduler()
    if args.mode == "F":
        sched.enabled = False
    else:
        sched.enable()
    sched.configure_allreduce(enabled=args.mode == "full", shared_dp_group=all_group, expert_dp_group=None,
                              gap_budgets={"moe_combine": 0.5, "moe_dispatch": 0.5, "attn_proj": 0.3, "attn_qkv": 0.3},
                              shared_ar_bw=3.0e8, expert_ar_bw=3.0e8)
    if args.mode != "F":
        model.setup_ar_buffer()
    extra = list(emb.parameters()) + list(final_norm.parameters()) + list(head.parameters())
    params = list(model.parameters()) + extra
    opt = torch.optim.AdamW(params, lr=1e-4, weight_decay=0.0, fused=True)
    # RoPE angles for the full sequence, Megatron layout [s, 1, 1, d]
    d = m["hidden"] // m["heads"]
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32, device=device) / d))
    fr = torch.outer(torch.arange(seq * world, dtype=torch.float32, device=device), inv)
    rotary = torch.cat([fr, fr], dim=-1).view(seq * world, 1, 1, d)
    n_batches = 4
    host = make_batches(torch, n_batches, seq, batch, m["vocab"], 100 + rank)
    dev_batches = [b.to(device) for b in host]
    last = {}

    trace = []
    converted = {"n": 0, "bytes": 0}

    def forward_loss(ids_full):
        ids, labels = ids_full[:-1], ids_full[1:]
        x = emb(ids)
        for layer in model.layers:
            x = layer(x, rotary)
        logits = head(final_norm(x))
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.reshape(-1))

    def train_step(ids_full):
        if args.forward_only:
            with torch.no_grad():
                return forward_loss(ids_full)
        for p in params:
            p.grad = None
            if hasattr(p, "_ar_buf_written"):
                p._ar_buf_written = False
        loss = forward_loss(ids_full)
        loss.backward()
        sched.finish_batch()
        if world > 1:
            for p in extra:
                if p.grad is not None:
                    p.grad.div_(world)
                    dist.all_reduce(p.grad, group=all_group)
        # The reference's flat buffers hold gradients in the parameter's dtype (its default,
        # accumulate_in_fp32=False), so handing them to the optimizer is a pointer assignment; a
        # dtype conversion, should one ever be needed, is counted and reported in the config record.
        converted["n"] = converted["bytes"] = 0
        for p in model.parameters():
            mg = getattr(p, "main_grad", None)
            if mg is not None and getattr(p, "_ar_buf_written", False):
                if mg.dtype == p.dtype:
                    p.grad = mg
                else:
                    p.grad = mg.to(p.dtype)
                    converted["n"] += 1
                    converted["bytes"] += mg.numel() * mg.element_size()
        opt.step()
        sched.clear_iteration()
        return loss

    def step_device(i):
        last["loss"] = train_step(dev_batches[i % n_batches])

    reader = LossReader(torch, args.steps)

    def step_e2e(i):
        ids = host[i % n_batches].to(device, non_blocking=True)
        reader.submit(i, train_step(ids))

    try:
        for i in range(args.warmup):
            step_device(i)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        emit(rank, {"impl": "reference", "unavailable": f"reference step failed: {type(e).__name__}: {e}"[:400]})
        return
    if args.profile:
        _profile_one_step(torch, step_device, args.profile, rank)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, _ = timed_region(torch, dist, world, step_device, args.steps)
    _, wall_e2e = timed_region(torch, dist, world, step_e2e, args.steps)
    assert len(reader.values) == args.steps, "every step's loss is read on the host inside the timed region"
    last["loss_val"] = reader.values[-1]
    trace.extend(reader.values)
    clocks = sampler.stop() if rank == 0 else {}
    tokens = world * seq * batch * args.steps
    value = tokens / (ms / 1e3)
    emit(rank, {
        "metric": METRIC_FWD if args.forward_only else METRIC_TRAIN,
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
        "impl": "reference",
        "config": {"model": "reference TransformerLayer x%d, hidden %d, %d/%d heads, 8 experts top-2 GELU ffn %d "
                            "(FLOP-matched to SwiGLU %d), LayerNorm, vocab %d; embedding / head / loss / AdamW from torch"
                            % (args.layers, m["hidden"], m["heads"], m["kv_heads"], ffn_ref, m["ffn"], m["vocab"]),
                   "arch": "matched", "forward_only": bool(args.forward_only),
                   "global_batch": batch, "seq_len": seq * world, "seq_per_rank": seq,
                   "parallelism": f"sp{world}ep{world}", "scheduler_mode": args.mode, "dx_chunks": args.chunks,
                   "grad_dtype_conversions_per_step": converted["n"], "grad_bytes_converted_per_step": converted["bytes"],
                   "loss": float(last["loss_val"]), **({"loss_trace": trace} if args.loss_trace else {})},
        "clocks": clocks,
        "e2e": {"value": tokens / (wall_e2e / 1e3), "unit": "tokens/s", "ms_per_step": wall_e2e / args.steps,
                "h2d_bytes_per_step": (seq + 1) * batch * 8, "d2h_bytes_per_step": 4,
                "loss_readback": "copied to pinned memory behind every step, read on the host one step later (last step at the end of the loop)"},
        "gpu_launches": 0,
    })
    dist.barrier()
    dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
