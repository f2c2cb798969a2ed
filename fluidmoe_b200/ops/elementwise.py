"""Front-ends of the memory-bound CUDA kernels (bf16 activations).  Callers reach these through
``ops.norm`` / ``ops.rope`` / ``ops.router`` / ``ops.permute`` / ``ops.optim``, which fall back to
PyTorch for CPU tensors and for dtypes the kernels do not cover."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native

LAUNCHES = 0


def _s() -> int:
    global LAUNCHES
    LAUNCHES += 1
    return _native.stream_ptr()


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _bf16(*ts) -> bool:
    return all(t is None or t.dtype == torch.bfloat16 for t in ts)


def norm_fwd(x, weight, bias, eps, kind):
    if not _bf16(x, weight, bias) or x.shape[-1] % 8 or not x.is_contiguous():
        return None
    T, H = x.shape
    y = torch.empty_like(x)
    ln = kind == "layernorm"
    mean = torch.empty(T, dtype=torch.float32, device=x.device) if ln else None
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    _native.lib().norm_fwd(x.data_ptr(), weight.data_ptr(), _ptr(bias), y.data_ptr(), _ptr(mean),
                           rstd.data_ptr(), T, H, float(eps), 0 if ln else 1, _s())
    return y, mean, rstd


def norm_bwd(dy, x, weight, mean, rstd, kind, has_bias, residual_grad):
    if not _bf16(dy, x, weight, residual_grad) or x.shape[-1] % 8 or x.shape[-1] > 8192:
        return None
    T, H = x.shape
    lib = _native.lib()
    dy = dy.contiguous()
    dx = torch.empty_like(x)
    nb = lib.norm_bwd_blocks(T)
    partial = torch.empty(nb, 2, H, dtype=torch.float32, device=x.device)
    dw = torch.empty(H, dtype=torch.float32, device=x.device)
    db = torch.empty(H, dtype=torch.float32, device=x.device) if has_bias else None
    ln = kind == "layernorm"
    lib.norm_bwd(dy.data_ptr(), x.data_ptr(), weight.data_ptr(), _ptr(mean) if ln else 0, rstd.data_ptr(),
                 _ptr(residual_grad.contiguous() if residual_grad is not None else None), dx.data_ptr(),
                 partial.data_ptr(), dw.data_ptr(), _ptr(db), T, H, 0 if ln else 1, _s())
    return dx, dw, db


_ROPE_TABLES = {}


def _cos_sin_table(freqs, rot):
    """``[positions, rot, 2]`` fp32 (cos, sin) of the angle tensor, computed once per angle tensor
    (keyed by storage address, shape and in-place version; a few entries are kept)."""
    key = (freqs.data_ptr(), tuple(freqs.shape), freqs._version, str(freqs.device))
    tab = _ROPE_TABLES.get(key)
    if tab is None:
        f = freqs.reshape(-1, rot).to(torch.float32)
        tab = torch.stack((torch.cos(f), torch.sin(f)), dim=-1).contiguous()
        if len(_ROPE_TABLES) >= 8:
            _ROPE_TABLES.pop(next(iter(_ROPE_TABLES)))
        _ROPE_TABLES[key] = tab
    return tab


def rope_packed_(qkv, freqs, q_per_group, head_dim, backward, wait=None):
    s, b, G, gs = qkv.shape
    rot = freqs.shape[-1]
    if qkv.dtype != torch.bfloat16 or rot % 16 or not qkv.is_contiguous():
        return None
    f = _cos_sin_table(freqs, rot)
    assert f.shape[0] >= s
    if wait is None:
        _native.lib().rope_packed(qkv.data_ptr(), f.data_ptr(), s * b * G, q_per_group + 2, q_per_group + 1,
                                  head_dim, rot, b * G, int(backward), _s())
    else:
        _native.lib().rope_packed_gated(qkv.data_ptr(), f.data_ptr(), s * b * G, q_per_group + 2, q_per_group + 1,
                                        head_dim, rot, b * G, int(backward), wait["flags"], wait["n"],
                                        wait["expected"], wait["wait_ns"], wait["timeout_ns"], wait["status"], _s())
    return qkv


def topk_softmax(logits, top_k):
    T, E = logits.shape
    logits = logits.contiguous()
    idx = torch.empty(T, top_k, dtype=torch.int64, device=logits.device)
    probs = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    _native.lib().topk_softmax(logits.data_ptr(), idx.data_ptr(), probs.data_ptr(), T, E, top_k, _s())
    return idx, probs


def gather_rows(x, idx, out=None):
    if x.dtype != torch.bfloat16 or x.shape[1] % 8 or not x.is_contiguous():
        return None
    idx = idx.to(torch.int64).contiguous()
    if out is None:
        out = torch.empty(idx.numel(), x.shape[1], dtype=x.dtype, device=x.device)
    _native.lib().gather_rows(x.data_ptr(), idx.data_ptr(), out.data_ptr(), idx.numel(), x.shape[1], _s())
    return out


def unpermute_reduce(rows, slot_of_token, residual=None, wait=None):
    """``wait`` (``dict(flags, n, expected, wait_ns, timeout_ns, status)``, addresses as ints): the
    kernel first waits, bounded, until the ``n`` per-source arrival counters at ``flags`` have
    reached ``expected`` (rows that peers push into ``rows``)."""
    if rows.dtype != torch.bfloat16 or rows.shape[1] % 8 or not rows.is_contiguous() or slot_of_token.shape[1] > 16:
        return None
    T, k = slot_of_token.shape
    H = rows.shape[1]
    slot = slot_of_token.to(torch.int32).contiguous()
    if residual is not None:
        residual = residual.contiguous()
        assert residual.dtype == torch.bfloat16
    out = torch.empty(T, H, dtype=rows.dtype, device=rows.device)
    if wait is None:
        _native.lib().unpermute_reduce(rows.data_ptr(), slot.data_ptr(), _ptr(residual), out.data_ptr(), T, k, H, _s())
    else:
        _native.lib().unpermute_reduce_gated(rows.data_ptr(), slot.data_ptr(), _ptr(residual), out.data_ptr(), T, k,
                                             H, wait["flags"], wait["n"], wait["expected"], wait["wait_ns"],
                                             wait["timeout_ns"], wait["status"], _s())
    return out


def _same_cuda_device(p, *others) -> None:
    """The kernels below take raw addresses: every operand must live on the parameter's GPU."""
    if not p.is_cuda:
        raise ValueError("native optimizer kernels need CUDA tensors")
    for t in others:
        if t is not None and (not t.is_cuda or t.device != p.device):
            raise ValueError(f"optimizer operand on {t.device}, parameter on {p.device}: load optimizer state "
                             "with FusedAdam.load_state_dict, which moves it to the parameter's device")


def adam_step(p, master, g, m, v, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, zero_grad=False):
    assert p.dtype == torch.bfloat16 and g.dtype == torch.float32 and m.dtype == v.dtype
    _same_cuda_device(p, master, g, m, v)
    _native.lib().adam(p.data_ptr(), _ptr(master), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(),
                       float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), int(step),
                       float(grad_scale), int(zero_grad), int(m.dtype == torch.bfloat16), _s())


def adam_background(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, num_ctas=0, stream=None):
    """Adam on bf16 parameter / bf16 moments / fp32 gradient with the small-CTA kernel that fits on
    an SM beside a resident tensor-core kernel.  ``stream`` is the raw stream handle to launch on."""
    global LAUNCHES
    assert p.dtype == torch.bfloat16 and m.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and g.dtype == torch.float32
    _same_cuda_device(p, g, m, v)
    LAUNCHES += 1
    _native.lib().adam_background(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), float(lr),
                                  float(beta1), float(beta2), float(eps), float(weight_decay), int(step),
                                  float(grad_scale), int(num_ctas), _s() if stream is None else stream)


def moe_plan(top_idx, top_probs, num_experts, capacity):
    """Padded-capacity routing plan on the device (one CTA per expert, no sort, no host sync)."""
    T, k = top_idx.shape
    dev = top_idx.device
    top_idx = top_idx.contiguous()
    top_probs = top_probs.float().contiguous()
    sorted_indices = torch.empty(num_experts * capacity, dtype=torch.int64, device=dev)
    slot_probs = torch.empty(num_experts * capacity, dtype=torch.float32, device=dev)
    slot_of_token = torch.empty(T, k, dtype=torch.int32, device=dev)
    routed = torch.empty(num_experts, dtype=torch.int32, device=dev)
    _native.lib().moe_plan(top_idx.data_ptr(), top_probs.data_ptr(), T, k, num_experts, capacity,
                           sorted_indices.data_ptr(), slot_probs.data_ptr(), slot_of_token.data_ptr(),
                           routed.data_ptr(), _s())
    return sorted_indices, slot_probs, slot_of_token, routed


def cross_entropy_(logits, labels, grad_scale):
    """In place: returns per-row losses (fp32) and leaves ``(softmax - onehot) * grad_scale`` in
    ``logits`` (bf16 [T, V], V a multiple of 8)."""
    T, V = logits.shape
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    _native.lib().cross_entropy(logits.data_ptr(), labels.contiguous().data_ptr(), loss.data_ptr(), T, V,
                                float(grad_scale), _s())
    return loss
