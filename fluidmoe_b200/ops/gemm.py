"""tcgen05 GEMM front-end (dense, grouped-M and grouped-K weight-gradient shapes).

Each function has a pure-PyTorch fp32-accumulating fallback that is used for CPU tensors (the
gloo test path) and doubles as the numerical oracle for the CUDA kernel.  The grouped variants
are the counterpart of the reference's ``grouped_fc1_act`` / ``grouped_fc2`` / ``grouped_fc1_dx``
/ ``grouped_fc2_dx`` helpers (fluid/moe/forward.py:217-352, fluid/moe/backward.py:400-480).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native

_STATUS = {}
LAUNCHES = 0  # number of native kernel launches issued by this module (bench bookkeeping)


def status_buffer(device) -> torch.Tensor:
    key = str(device)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(8, dtype=torch.int32, device=device)
    return _STATUS[key]


class FluidKernelTimeout(RuntimeError):
    """A device-side bounded wait ran out; the kernel returned instead of hanging."""


def check_status(device=None) -> None:
    """Read the status words (host sync) and raise if a kernel reported a timeout."""
    for key, buf in _STATUS.items():
        if device is not None and key != str(device):
            continue
        vals = buf.tolist()
        if vals[0] != 0:
            buf.zero_()
            raise FluidKernelTimeout(
                f"kernel {vals[1]} block {vals[2]} gave up: code={vals[0]} what={vals[3]} "
                f"expected={vals[4]} observed={vals[5]}"
            )


CTA_PAIR = int(__import__("os").environ.get("FLUIDMOE_GEMM_CTA_PAIR", "1"))


def _launch(desc: dict) -> None:
    global LAUNCHES
    LAUNCHES += 1
    desc.setdefault("cta_pair", CTA_PAIR)
    _native.lib().gemm_launch(desc, _native.stream_ptr())


def _operand(t: torch.Tensor):
    assert t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1, (t.dtype, t.shape, t.stride())
    return t.data_ptr(), t.shape[1], t.shape[0], t.stride(0)


def _pick_bn(n: int) -> int:
    return 256 if n > 128 else 128


def _group_kw(group_rows, group_offs, uniform_rows, group_b=None):
    kw = {"uniform_rows": int(uniform_rows)}
    if group_rows is not None:
        assert group_rows.dtype == torch.int32 and group_offs.dtype == torch.int32
        kw["group_rows"] = group_rows.data_ptr()
        kw["group_offs"] = group_offs.data_ptr()
        kw["num_groups"] = group_rows.numel()
    if group_b is not None:
        assert group_b.dtype == torch.int32
        kw["group_b"] = group_b.data_ptr()
    return kw


# --------------------------------------------------------------------------------------------
# reference (CPU / oracle) helpers
# --------------------------------------------------------------------------------------------
def _groups(rows_total, num_groups, group_rows, group_offs, uniform_rows, group_b=None):
    """List of (B index, row offset, rows) per group."""
    if group_rows is None:
        return [(g, g * uniform_rows, uniform_rows) for g in range(num_groups)]
    r, o = group_rows.tolist(), group_offs.tolist()
    b = group_b.tolist() if group_b is not None else list(range(len(r)))
    return [(b[g], o[g], r[g]) for g in range(len(r))]


def _b_mat(b: torch.Tensor, g: int, b_layout: str) -> torch.Tensor:
    """Return group g of B as a [K, N] matrix."""
    bg = b[g] if b.dim() == 3 else b
    return bg if b_layout == "kn" else bg.t()


def act_ref(x: torch.Tensor, kind: str) -> torch.Tensor:
    if kind == "gelu":
        return torch.nn.functional.gelu(x)
    if kind == "silu":
        return torch.nn.functional.silu(x)
    if kind == "swiglu":
        g, u = x.chunk(2, dim=-1)
        return torch.nn.functional.silu(g) * u
    if kind == "none":
        return x
    raise ValueError(kind)


# --------------------------------------------------------------------------------------------
# public ops
# --------------------------------------------------------------------------------------------
def grouped_gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    b_layout: str = "kn",
    group_rows: Optional[torch.Tensor] = None,
    group_offs: Optional[torch.Tensor] = None,
    uniform_rows: Optional[int] = None,
    group_b: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
    accumulate: bool = False,
    alpha: float = 1.0,
    gate: Optional[dict] = None,
    max_ctas: int = 0,
) -> torch.Tensor:
    """``out[rows_g] = a[rows_g] @ B_g`` for every group g.

    a: [rows, K] bf16.  b: [G, K, N] (``b_layout='kn'``) or [G, N, K] (``'nk'``); a 2-D b is one
    group.  Rows of group g are ``[group_offs[g], group_offs[g] + group_rows[g])`` (device int32
    tensors, no host sync) or ``uniform_rows`` consecutive rows per group.
    """
    b3 = b if b.dim() == 3 else b.unsqueeze(0)
    G = b3.shape[0]
    K = a.shape[1]
    N = b3.shape[2] if b_layout == "kn" else b3.shape[1]
    if uniform_rows is None and group_rows is None:
        assert G == 1
        uniform_rows = a.shape[0]
    out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is None:
        out = torch.zeros(a.shape[0], N, dtype=out_dtype, device=a.device) if group_rows is not None \
            else torch.empty(a.shape[0], N, dtype=out_dtype, device=a.device)
    if not _native.use_native(a, b):
        for g, o, r in _groups(a.shape[0], G, group_rows, group_offs, uniform_rows, group_b):
            if r == 0:
                continue
            res = alpha * (a[o:o + r].float() @ _b_mat(b3, g, b_layout).float())
            out[o:o + r] = (out[o:o + r].float() + res if accumulate else res).to(out.dtype)
        return out
    assert K % 8 == 0 and N % 8 == 0
    b2 = b3.reshape(-1, b3.shape[2])
    ap, ai, ao, lda = _operand(a)
    bp, bi, bo, ldb = _operand(b2)
    desc = dict(
        A=ap, a_inner=ai, a_outer=ao, lda=lda, a_mn=0,
        B=bp, b_inner=bi, b_outer=bo, ldb=ldb, b_mn=1 if b_layout == "kn" else 0,
        mode=0, num_groups=G, M=a.shape[0], N=N, K=K, b_group_stride=b3.shape[1],
        bn=_pick_bn(N), epi=0, C=out.data_ptr(), ldc=out.stride(0),
        out_fp32=int(out.dtype == torch.float32), accumulate=int(accumulate), alpha=float(alpha),
        max_ctas=max_ctas, status=status_buffer(a.device).data_ptr(),
    )
    desc.update(_group_kw(group_rows, group_offs, uniform_rows or 0, group_b))
    if gate:
        desc.update(gate)
    _launch(desc)
    return out


def gemm_nt(a: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
    """a[M,K] @ w[N,K]^T (the nn.Linear shape)."""
    return grouped_gemm(a, w, b_layout="nk", **kw)


def gemm_nn(a: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
    """a[M,K] @ w[K,N]."""
    return grouped_gemm(a, w, b_layout="kn", **kw)


def grouped_gemm_act(
    a: torch.Tensor,
    w: torch.Tensor,
    probs: Optional[torch.Tensor],
    *,
    activation: str = "gelu",
    group_rows=None,
    group_offs=None,
    uniform_rows=None,
    group_b=None,
    save_pre: bool = True,
    gate: Optional[dict] = None,
    act_out: Optional[torch.Tensor] = None,
    pre_out: Optional[torch.Tensor] = None,
):
    """Expert FC1 with the activation and the routing probability fused into the epilogue.

    a: [rows, H]; w: [G, H, F] (or [G, H, 2F] for ``activation='swiglu'``, gate half first);
    probs: fp32 [rows] or None.  Returns ``(act * prob [rows, F], pre-activation or None)``.
    """
    G, H, Fw = w.shape
    gated = activation == "swiglu"
    F = Fw // 2 if gated else Fw
    rows = a.shape[0]
    if uniform_rows is None and group_rows is None:
        assert G == 1
        uniform_rows = rows
    if not _native.use_native(a, w):
        act = act_out if act_out is not None else torch.zeros(rows, F, dtype=a.dtype, device=a.device)
        pre = pre_out if pre_out is not None else (
            torch.zeros(rows, Fw, dtype=a.dtype, device=a.device) if save_pre else None)
        for g, o, r in _groups(rows, G, group_rows, group_offs, uniform_rows, group_b):
            if r == 0:
                continue
            x = a[o:o + r].float() @ w[g].float()
            if save_pre:
                pre[o:o + r] = x.to(a.dtype)
            y = act_ref(x, activation)
            if probs is not None:
                y = y * probs[o:o + r].float().unsqueeze(1)
            act[o:o + r] = y.to(a.dtype)
        return act, pre
    zeros_needed = group_rows is not None
    alloc = torch.zeros if zeros_needed else torch.empty
    act = act_out if act_out is not None else alloc(rows, F, dtype=a.dtype, device=a.device)
    pre = pre_out if pre_out is not None else (
        alloc(rows, Fw, dtype=a.dtype, device=a.device) if save_pre else None)
    w2 = w.reshape(G * H, Fw)
    ap, ai, ao, lda = _operand(a)
    bp, bi, bo, ldb = _operand(w2)
    lib = _native.lib()
    kind = {"gelu": lib.ACT_GELU, "silu": lib.ACT_SILU, "swiglu": lib.ACT_SILU, "none": lib.ACT_NONE}[activation]
    desc = dict(
        A=ap, a_inner=ai, a_outer=ao, lda=lda, a_mn=0,
        B=bp, b_inner=bi, b_outer=bo, ldb=ldb, b_mn=1,
        mode=0, num_groups=G, M=rows, N=F, K=H, b_group_stride=H,
        gated=int(gated), n_half=F, bn=256 if (gated or F > 128) else 128, epi=lib.EPI_ACT,
        act_out=act.data_ptr(), ld_act=act.stride(0),
        pre_out=pre.data_ptr() if pre is not None else 0, ld_pre=Fw,
        probs=probs.data_ptr() if probs is not None else 0, act_kind=kind,
        status=status_buffer(a.device).data_ptr(),
    )
    desc.update(_group_kw(group_rows, group_offs, uniform_rows or 0, group_b))
    if probs is not None:
        assert probs.dtype == torch.float32 and probs.is_contiguous()
    if gate:
        desc.update(gate)
    _launch(desc)
    return act, pre


def grouped_gemm_dact(
    dy: torch.Tensor,
    w2: torch.Tensor,
    pre: torch.Tensor,
    probs: Optional[torch.Tensor],
    *,
    activation: str = "gelu",
    group_rows=None,
    group_offs=None,
    uniform_rows=None,
    group_b=None,
    gate: Optional[dict] = None,
    dpre_out: Optional[torch.Tensor] = None,
    dprobs_out: Optional[torch.Tensor] = None,
):
    """Backward of FC2 and of ``act * prob`` in one kernel.

    dy: [rows, H] gradient of the FC2 output; w2: [G, F, H]; pre: saved FC1 pre-activation
    ([rows, F] or [rows, 2F]).  Returns ``(dpre, dprobs fp32 [rows])`` where
    ``dActW = dy @ w2^T``, ``dprobs = sum_F(dActW * act(pre))`` and
    ``dpre = dActW * prob * act'(pre)`` (fluid/moe/backward.py:341-356).
    """
    G, F, H = w2.shape
    gated = activation == "swiglu"
    rows = dy.shape[0]
    if uniform_rows is None and group_rows is None:
        assert G == 1
        uniform_rows = rows
    if not _native.use_native(dy, w2):
        dpre = dpre_out if dpre_out is not None else torch.zeros_like(pre)
        dprobs = dprobs_out if dprobs_out is not None else torch.zeros(rows, dtype=torch.float32, device=dy.device)
        for g, o, r in _groups(rows, G, group_rows, group_offs, uniform_rows, group_b):
            if r == 0:
                continue
            dactw = dy[o:o + r].float() @ w2[g].float().t()
            x = pre[o:o + r].float().detach().requires_grad_(True)
            with torch.enable_grad():
                a_ = act_ref(x, activation)
            dprobs[o:o + r] = (dactw * a_.detach()).sum(-1)
            p = probs[o:o + r].float().unsqueeze(1) if probs is not None else 1.0
            (gx,) = torch.autograd.grad(a_, x, dactw * p)
            dpre[o:o + r] = gx.to(dpre.dtype)
        return dpre, dprobs
    bn = _pick_bn(F)
    nt = (F + bn - 1) // bn
    alloc = torch.zeros if group_rows is not None else torch.empty
    dpre = dpre_out if dpre_out is not None else alloc(pre.shape, dtype=pre.dtype, device=pre.device)
    partial = torch.zeros(rows, nt * 2, dtype=torch.float32, device=dy.device)
    wflat = w2.reshape(G * F, H)
    ap, ai, ao, lda = _operand(dy)
    bp, bi, bo, ldb = _operand(wflat)
    lib = _native.lib()
    kind = {"gelu": lib.ACT_GELU, "silu": lib.ACT_SILU, "swiglu": lib.ACT_SILU, "none": lib.ACT_NONE}[activation]
    desc = dict(
        A=ap, a_inner=ai, a_outer=ao, lda=lda, a_mn=0,
        B=bp, b_inner=bi, b_outer=bo, ldb=ldb, b_mn=0,
        mode=0, num_groups=G, M=rows, N=F, K=H, b_group_stride=F,
        gated=int(gated), n_half=F, bn=bn, epi=lib.EPI_DACT,
        C=dpre.data_ptr(), ldc=dpre.stride(0), pre_in=pre.data_ptr(), ld_pre_in=pre.stride(0),
        probs=probs.data_ptr() if probs is not None else 0, dprobs=partial.data_ptr(), act_kind=kind,
        status=status_buffer(dy.device).data_ptr(),
    )
    desc.update(_group_kw(group_rows, group_offs, uniform_rows or 0, group_b))
    if gate:
        desc.update(gate)
    _launch(desc)
    dprobs = partial.sum(dim=1)
    if dprobs_out is not None:
        # rows outside the groups touched by this call keep their previous value
        if group_rows is None and uniform_rows * G == rows:
            dprobs_out.copy_(dprobs)
        else:
            dprobs_out.add_(dprobs)
        return dpre, dprobs_out
    return dpre, dprobs


def grouped_gemm_wgrad(
    a: torch.Tensor,
    dy: torch.Tensor,
    num_groups: int = 1,
    *,
    group_rows=None,
    group_offs=None,
    uniform_rows=None,
    out: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    alpha: float = 1.0,
    max_ctas: int = 0,
) -> torch.Tensor:
    """``out[g] (+)= a[rows_g]^T @ dy[rows_g]`` -> [G, M, N] (weight-gradient shape).

    Rows between the end of a group and the next multiple of 64 must be zero in ``a`` or ``dy``
    (the contraction runs in 64-row blocks); group offsets must be multiples of 64 or the
    groups must tile the buffer exactly.  fp32 ``out`` with ``accumulate=True`` adds straight
    into a gradient buffer (fluid/moe/backward.py:541-573, fluid/core/scheduler.py:188-213).
    """
    rows, M = a.shape
    N = dy.shape[1]
    G = num_groups
    if uniform_rows is None and group_rows is None:
        assert G == 1
        uniform_rows = rows
    if out is None:
        out = torch.zeros(G, M, N, dtype=torch.float32, device=a.device)
        accumulate = False
    o3 = out.view(G, M, N)
    if not _native.use_native(a, dy):
        for g, o, r in _groups(rows, G, group_rows, group_offs, uniform_rows):
            res = alpha * (a[o:o + r].float().t() @ dy[o:o + r].float())
            o3[g] = (o3[g].float() + res if accumulate else res).to(out.dtype)
        return out
    assert M % 8 == 0 and N % 8 == 0 and out.is_contiguous()
    ap, ai, ao, lda = _operand(a)
    bp, bi, bo, ldb = _operand(dy)
    desc = dict(
        A=ap, a_inner=ai, a_outer=ao, lda=lda, a_mn=1,
        B=bp, b_inner=bi, b_outer=bo, ldb=ldb, b_mn=1,
        mode=1, num_groups=G, M=M, N=N, K=0, bn=_pick_bn(N), epi=0,
        C=out.data_ptr(), ldc=N, c_group_stride=M * N,
        out_fp32=int(out.dtype == torch.float32), accumulate=int(accumulate), alpha=float(alpha),
        max_ctas=max_ctas, status=status_buffer(a.device).data_ptr(),
    )
    kw = _group_kw(group_rows, group_offs, uniform_rows or 0)
    kw.pop("num_groups", None)
    desc.update(kw)
    _launch(desc)
    return out


def grouped_gemm_wgrad_adam(
    a: torch.Tensor,
    dy: torch.Tensor,
    num_groups: int,
    param: torch.Tensor,
    exp_avg: torch.Tensor,
    exp_avg_sq: torch.Tensor,
    *,
    lr: float,
    beta1: float,
    beta2: float,
    eps: float,
    weight_decay: float,
    step: int,
    grad_scale: float = 1.0,
    group_rows=None,
    group_offs=None,
    uniform_rows=None,
    max_ctas: int = 0,
) -> None:
    """Weight gradient with the optimizer in the epilogue: ``g[g] = a[rows_g]^T @ dy[rows_g]`` is
    never written; the AdamW update of ``param[g]`` ([G, M, N] bf16, moments bf16) is applied to
    each output tile while it is still in TMEM.  Valid only when this GEMM produces the complete
    gradient of the step (one micro-batch, no data-parallel reduction of ``param``).  The
    reference stores the gradient (fluid/moe/backward.py:541-573) and runs the optimizer later."""
    rows, M = a.shape
    N = dy.shape[1]
    G = num_groups
    if uniform_rows is None and group_rows is None:
        assert G == 1
        uniform_rows = rows
    rbc1 = 1.0 / (1.0 - beta1 ** step)
    rbc2 = 1.0 / (1.0 - beta2 ** step)
    p3, m3, v3 = param.view(G, M, N), exp_avg.view(G, M, N), exp_avg_sq.view(G, M, N)
    if not (_native.use_native(a, dy) and param.dtype == torch.bfloat16 and exp_avg.dtype == torch.bfloat16):
        for g, o, r in _groups(rows, G, group_rows, group_offs, uniform_rows):
            gr = grad_scale * (a[o:o + r].float().t() @ dy[o:o + r].float())
            m = m3[g].float().mul_(beta1).add_(gr, alpha=1 - beta1)
            v = v3[g].float().mul_(beta2).addcmul_(gr, gr, value=1 - beta2)
            w = p3[g].float()
            w = w - lr * ((m * rbc1) / ((v * rbc2).sqrt() + eps) + weight_decay * w)
            m3[g].copy_(m)
            v3[g].copy_(v)
            p3[g].copy_(w)
        return
    assert M % 8 == 0 and N % 8 == 0 and param.is_contiguous() and exp_avg.is_contiguous() and exp_avg_sq.is_contiguous()
    for t in (param, exp_avg, exp_avg_sq):
        # raw addresses go to the kernel: a host tensor here (moments loaded from a checkpoint
        # without moving them) would be dereferenced on the device
        if not t.is_cuda or t.device != a.device:
            raise ValueError(f"optimizer operand on {t.device}, activations on {a.device}")
    ap, ai, ao, lda = _operand(a)
    bp, bi, bo, ldb = _operand(dy)
    desc = dict(
        A=ap, a_inner=ai, a_outer=ao, lda=lda, a_mn=1,
        B=bp, b_inner=bi, b_outer=bo, ldb=ldb, b_mn=1,
        mode=1, num_groups=G, M=M, N=N, K=0, bn=_pick_bn(N), epi=_native.lib().EPI_ADAM,
        ldc=N, c_group_stride=M * N, alpha=float(grad_scale),
        adam_p=param.data_ptr(), adam_m=exp_avg.data_ptr(), adam_v=exp_avg_sq.data_ptr(),
        adam_lr=float(lr), adam_beta1=float(beta1), adam_beta2=float(beta2), adam_eps=float(eps),
        adam_wd=float(weight_decay), adam_rbc1=float(rbc1), adam_rbc2=float(rbc2),
        max_ctas=max_ctas, status=status_buffer(a.device).data_ptr(),
    )
    kw = _group_kw(group_rows, group_offs, uniform_rows or 0)
    kw.pop("num_groups", None)
    desc.update(kw)
    _launch(desc)
