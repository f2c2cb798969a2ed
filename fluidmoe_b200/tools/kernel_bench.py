"""Single-kernel benchmarks with roofline fractions (one GPU).

    python -m fluidmoe_b200.tools.kernel_bench gemm --m 8192 --n 8192 --k 4096
    python -m fluidmoe_b200.tools.kernel_bench all

Each case warms up, flushes L2 between timed launches (writes a 256 MB buffer), times with CUDA
events and prints milliseconds, achieved TFLOP/s or GB/s and the fraction of the measured peaks in
``MEASURED_PEAKS.json`` at the repository root (cuBLAS bf16 burst throughput and copy bandwidth);
without that file the fallback peaks 1590 TFLOP/s and 6650 GB/s are used and labelled as such.
The same cases, run small, are what the ncu summaries under ``profiles/`` were captured from.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from ..ops import elementwise as ew
from ..ops import flash, gemm, norm, permute, rope, router

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        with open(os.path.join(_ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["bf16_tflops"], p["hbm_gbs"], "of measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 6650.0, "of fallback"


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    gemm.check_status()
    return total / iters


def report(name, ms, flops=0.0, bytes_=0.0):
    tf, gb, label = peaks()
    parts = [f"{name:34s} {ms:9.4f} ms"]
    if flops:
        t = flops / ms / 1e9
        parts.append(f"{t:8.1f} TFLOP/s ({t / tf:5.2f} {label} cuBLAS bf16)")
    if bytes_:
        g = bytes_ / ms / 1e6
        parts.append(f"{g:8.1f} GB/s ({g / gb:5.2f} {label} copy bandwidth)")
    try:
        print("  ".join(parts), flush=True)
    except BrokenPipeError:      # output piped into `head`
        pass


def _r(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def case_gemm(a):
    x, w = _r(a.m, a.k), _r(a.n, a.k)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    report(f"gemm nk {a.m}x{a.n}x{a.k}", timed(lambda: gemm.grouped_gemm(x, w, b_layout="nk", out=out)),
           2.0 * a.m * a.n * a.k)
    report("  cuBLAS (torch.matmul) same shape", timed(lambda: torch.matmul(x, w.t(), out=out)), 2.0 * a.m * a.n * a.k)


def case_fc1(a):
    R, H, F, G = a.rows, a.hidden, a.ffn, a.experts
    x, w = _r(R, H), _r(G, H, 2 * F, scale=0.02)
    probs = torch.rand(R, device="cuda")
    act = torch.empty(R, F, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty(R, 2 * F, device="cuda", dtype=torch.bfloat16)
    report(f"fc1 swiglu*prob G={G} {R}x{H}x{2 * F}",
           timed(lambda: gemm.grouped_gemm_act(x, w, probs, activation="swiglu", uniform_rows=R // G,
                                               act_out=act, pre_out=pre)), 2.0 * R * H * 2 * F)
    return x, w, probs, act, pre


def case_dact(a):
    R, H, F, G = a.rows, a.hidden, a.ffn, a.experts
    dy, w2, pre = _r(R, H), _r(G, F, H, scale=0.02), _r(R, 2 * F)
    probs = torch.rand(R, device="cuda")
    dpre = torch.empty_like(pre)
    report(f"fc2-dX + dact G={G} {R}x{F}x{H}",
           timed(lambda: gemm.grouped_gemm_dact(dy, w2, pre, probs, activation="swiglu", uniform_rows=R // G,
                                                dpre_out=dpre)), 2.0 * R * H * F)


def case_wgrad(a):
    R, H, F, G = a.rows, a.hidden, a.ffn, a.experts
    x, dy = _r(R, H), _r(R, 2 * F)
    out = torch.zeros(G, H, 2 * F, device="cuda")
    report(f"wgrad fp32 G={G} {H}x{2 * F}, K={R // G}",
           timed(lambda: gemm.grouped_gemm_wgrad(x, dy, G, uniform_rows=R // G, out=out, accumulate=False)),
           2.0 * R * H * 2 * F, bytes_=out.numel() * 4.0)


def case_wgrad_adam(a):
    """Expert weight gradient with the optimizer in the epilogue, against gradient store + Adam pass."""
    R, H, F, G = a.rows, a.hidden, a.ffn, a.experts
    x, dy = _r(R, H), _r(R, 2 * F)
    p = _r(G, H, 2 * F, scale=0.02)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    hyper = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1)
    fl, by = 2.0 * R * H * 2 * F, p.numel() * 12.0
    report(f"wgrad + Adam epilogue G={G} {H}x{2 * F}, K={R // G}",
           timed(lambda: gemm.grouped_gemm_wgrad_adam(x, dy, G, p, m, v, uniform_rows=R // G, **hyper)), fl, bytes_=by)
    out = torch.zeros(G, H, 2 * F, device="cuda")
    t1 = timed(lambda: gemm.grouped_gemm_wgrad(x, dy, G, uniform_rows=R // G, out=out, accumulate=False))
    t2 = timed(lambda: ew.adam_step(p.view(-1), None, out.view(-1), m.view(-1), v.view(-1), 1e-4, 0.9, 0.999, 1e-8, 0.0, 1))
    report("  gradient store (fp32) then Adam pass", t1 + t2, fl, bytes_=p.numel() * 20.0)
    report("    of which Adam pass", t2, bytes_=p.numel() * 16.0)


def case_flash(a):
    from ..ops import attention
    s, G, qpg, d = a.seq, a.kv_heads, a.q_per_kv, 128
    sc = 1.0 / math.sqrt(d)
    qkv = _r(s, 1, G, (qpg + 2) * d)
    fl = 4.0 * s * s * G * qpg * d / 2
    for ver in a.fwd_versions:
        report(f"flash fwd v{ver} causal s={s} heads={G * qpg}/{G}",
               timed(lambda: flash.flash_attn_fwd_packed(qkv, qpg, d, sc, version=ver)), fl)
    out, lse = flash.flash_attn_fwd_packed(qkv, qpg, d, sc)
    dout = torch.randn_like(out)
    for ver in a.bwd_versions:
        report(f"flash bwd v{ver} (delta + main + dq store)",
               timed(lambda: flash.flash_attn_bwd_packed(dout, qkv, out, lse, qpg, d, sc, version=ver)), 2.5 * fl)
    heads = qkv.view(s, 1, G, qpg + 2, d)
    q = heads[:, :, :, :qpg].reshape(s, 1, G * qpg, d).contiguous()
    k, v = heads[:, :, :, qpg].contiguous(), heads[:, :, :, qpg + 1].contiguous()
    report("  library fwd (cuDNN via torch), same shape", timed(lambda: attention._sdpa_fwd(q, k, v, sc, True)), fl)
    lo, ll = attention._sdpa_fwd(q, k, v, sc, True)
    report("  library bwd (cuDNN via torch), same shape",
           timed(lambda: attention._sdpa_bwd(dout, q, k, v, sc, True, lo, ll)), 2.5 * fl)


def case_norm(a):
    T, H = a.rows * 4, a.hidden
    x, w, dy = _r(T, H), _r(H), _r(T, H)
    y, mean, rstd = norm.norm_fwd(x, w, None, 1e-5, "rmsnorm")
    report(f"rmsnorm fwd {T}x{H}", timed(lambda: norm.norm_fwd(x, w, None, 1e-5, "rmsnorm")), bytes_=T * H * 4.0)
    report(f"rmsnorm bwd {T}x{H}", timed(lambda: norm.norm_bwd(dy, x, w, None, rstd, "rmsnorm", False, dy)),
           bytes_=T * H * 8.0)


def case_permute(a):
    T, H, E, k = a.rows * 2, a.hidden, 8, 2
    x = _r(T, H)
    ti, tp = router.topk_softmax(torch.randn(T, E, device="cuda"), k)
    cap = router.expert_capacity(T, k, E, 1.0)
    report(f"routing plan T={T} E={E} k={k}", timed(lambda: router.build_padded_plan(ti, tp, E, cap)))
    plan = router.build_padded_plan(ti, tp, E, cap)
    out = torch.empty(E * cap, H, device="cuda", dtype=torch.bfloat16)
    report(f"permute {E * cap}x{H}", timed(lambda: permute.permute_rows(x, plan.sorted_indices, out)),
           bytes_=E * cap * H * 4.0)
    report(f"unpermute-reduce {T}x{H} k={k}", timed(lambda: permute.unpermute_reduce(out, plan.slot_of_token, x)),
           bytes_=(E * cap + 2 * T) * H * 2.0)


def case_adam(a):
    n = a.elems
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    report(f"adam bf16 moments n={n}", timed(lambda: ew.adam_step(p, None, g, m, v, 1e-4, 0.9, 0.999, 1e-8, 0.0, 1)),
           bytes_=n * 16.0)


def case_ce(a):
    T, V = 4096, 32000
    logits = _r(T, V)
    labels = torch.randint(0, V, (T,), device="cuda")
    report(f"cross-entropy fwd+bwd {T}x{V}", timed(lambda: ew.cross_entropy_(logits, labels, 1.0 / T)),
           bytes_=T * V * 2.0 * 3)


def case_rope(a):
    s, G, qpg, d = a.seq, a.kv_heads, a.q_per_kv, 128
    qkv = _r(s, 1, G, (qpg + 2) * d)
    fr = rope.make_rope_freqs(s, d, device="cuda")
    report(f"rope packed s={s}", timed(lambda: rope.rope_packed_(qkv, fr, qpg, d)),
           bytes_=s * G * (qpg + 1) * d * 4.0)


def case_fused(a):
    """The device-initiated dispatch / combine kernels on one GPU: the only "peer" is this GPU
    itself, so the same kernels (peer-pointer tables, arrival counters, gated producer, scatter
    epilogue) run as on several GPUs, minus the NVLink hop."""
    from ..models.moe import EPPlan, MoEForwardState
    from ..parallel.fused import FusedCommContext

    T, H, F, E, k = a.rows // 2, a.hidden, a.ffn, a.experts if a.experts > 1 else 8, 2
    dev = torch.device("cuda", torch.cuda.current_device())
    ctx = FusedCommContext(None, 2 << 30, dev)
    plan = EPPlan(T, H, E, k, None, 1.0, torch.bfloat16, dev)

    class _L:
        layer_id, ffn_hidden_size = 0, F
    ctx.prepare(plan, None, _L)
    x = _r(T, H)
    ti, tp = router.topk_softmax(torch.randn(T, E, device="cuda"), k)
    rp = router.build_padded_plan(ti, tp, E, plan.expert_capacity)
    w1, w2 = _r(E, H, 2 * F, scale=0.02), _r(E, F, H, scale=0.02)
    b = ctx._buf(plan)
    rows = E * plan.expert_capacity

    def push():
        ctx._push(plan, x, rp.sorted_indices, rp.permuted_probs, b.tokens_em, b.probs_em, b.flags_fwd, b.bpg)

    def push_and_reset():
        push()
        b.flags_fwd.local.zero_()
    report(f"permute+dispatch (peer stores) {rows}x{H}", timed(push_and_reset), bytes_=rows * H * 4.0)

    def fc1():
        push()
        st = gemm.grouped_gemm_act(b.tokens_em.local, w1, b.probs_em.local, activation="swiglu",
                                   uniform_rows=plan.expert_capacity, gate=ctx._gate(b.flags_fwd, b.bpg))
        b.flags_fwd.local.zero_()
        return st
    report(f"dispatch + gated FC1 G={E} {rows}x{H}x{2 * F}", timed(fc1), 2.0 * rows * H * 2 * F)
    act, pre = fc1()
    state = MoEForwardState(b.tokens_em.local, b.probs_em.local, pre, act)

    def fc2():
        ctx._scatter_gemm(plan, state.act_em, w2, "kn", b.combined, b.cnt_combine_tbl)
        return ctx.unpermute(plan, b.combined.local, rp.slot_of_token, x)
    report(f"FC2 + combine (scatter epilogue) + unpermute {rows}x{F}x{H}", timed(fc2), 2.0 * rows * F * H)


def case_mma_issue(a):
    """Builds and runs the stand-alone MMA issue probe (``mma_issue_probe.cu`` next to this file)."""
    import subprocess
    import tempfile
    here = os.path.dirname(os.path.abspath(__file__))
    exe = os.path.join(tempfile.mkdtemp(), "mma_issue_probe")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.run([f"{cuda}/bin/nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
                    "-I", os.path.join(os.path.dirname(here), "csrc", "include"), "-o", exe,
                    os.path.join(here, "mma_issue_probe.cu"), "-lcuda"], check=True)
    print(subprocess.run([exe, "64"], check=True, capture_output=True, text=True).stdout, flush=True)


def case_softmax_pass(a):
    """Builds and runs the stand-alone probe of the softmax exponential pass (``softmax_pass_probe.cu``)."""
    import subprocess
    import tempfile
    here = os.path.dirname(os.path.abspath(__file__))
    exe = os.path.join(tempfile.mkdtemp(), "softmax_pass_probe")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.run([f"{cuda}/bin/nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", exe,
                    os.path.join(here, "softmax_pass_probe.cu")], check=True)
    print(subprocess.run([exe], check=True, capture_output=True, text=True).stdout, flush=True)


CASES = dict(mma_issue=case_mma_issue, softmax_pass=case_softmax_pass, gemm=case_gemm, fc1=case_fc1, dact=case_dact, wgrad=case_wgrad, wgrad_adam=case_wgrad_adam, flash=case_flash, norm=case_norm,
             permute=case_permute, adam=case_adam, ce=case_ce, rope=case_rope, fused=case_fused)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=list(CASES) + ["all"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=1)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--q-per-kv", type=int, default=4)
    ap.add_argument("--elems", type=int, default=1 << 28)
    ap.add_argument("--fwd-versions", type=int, nargs="+", default=[2, 1],
                    help="attention forward kernels to time (2: default; 20..24: share of polynomial exponentials; 1: first generation)")
    ap.add_argument("--bwd-versions", type=int, nargs="+", default=[2, 1])
    a = ap.parse_args(argv)
    torch.manual_seed(0)
    for name in (list(CASES) if a.case == "all" else [a.case]):
        CASES[name](a)


if __name__ == "__main__":
    main()
