"""Element-wise CUDA kernels against the PyTorch fp32 reference of the same op."""
import pytest
import torch

from fluidmoe_b200.ops import norm, permute, rope, router
from fluidmoe_b200.ops import elementwise as ew

pytestmark = pytest.mark.gpu


def _close(got, ref, tol=2e-2):
    got, ref = got.float().cpu(), ref.float().cpu()
    err = (got - ref).abs().max().item()
    assert err <= tol * (ref.abs().max().item() + 1e-6), (err, ref.abs().max().item())


@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm"])
@pytest.mark.parametrize("T,H", [(37, 256), (512, 4096), (5, 2048)])
def test_norm_fwd_bwd(kind, T, H):
    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    b = (0.1 * torch.randn(H, device="cuda")).bfloat16() if kind == "layernorm" else None
    dy = torch.randn(T, H, device="cuda").bfloat16()
    rg = torch.randn(T, H, device="cuda").bfloat16()
    y, mean, rstd = norm.norm_fwd(x, w, b, 1e-5, kind)
    dx, dw, db = norm.norm_bwd(dy, x, w, mean, rstd, kind, b is not None, rg)
    ry, rmean, rrstd = norm.norm_fwd(x.cpu().float(), w.cpu().float(), None if b is None else b.cpu().float(), 1e-5, kind)
    rdx, rdw, rdb = norm.norm_bwd(dy.cpu().float(), x.cpu().float(), w.cpu().float(), rmean, rrstd, kind,
                                  b is not None, rg.cpu().float())
    _close(y, ry)
    _close(rstd, rrstd, 1e-3)
    _close(dx, rdx)
    _close(dw, rdw)
    if db is not None:
        _close(db, rdb)


@pytest.mark.parametrize("backward", [False, True])
def test_rope_packed(backward):
    s, b, G, qpg, d = 64, 2, 2, 4, 128
    torch.manual_seed(1)
    qkv = torch.randn(s, b, G, (qpg + 2) * d, device="cuda").bfloat16()
    freqs = rope.make_rope_freqs(s, 64, device="cuda")
    ref = rope.rope_packed_(qkv.cpu().float().clone(), freqs.cpu(), qpg, d, backward)
    got = rope.rope_packed_(qkv.clone(), freqs, qpg, d, backward)
    _close(got, ref)


@pytest.mark.parametrize("E,k", [(8, 2), (64, 6)])
def test_topk_softmax(E, k):
    torch.manual_seed(2)
    logits = torch.randn(1000, E, device="cuda")
    idx, probs = ew.topk_softmax(logits, k)
    tl, ti = torch.topk(logits, k, dim=-1)
    assert torch.equal(idx, ti)
    _close(probs, torch.softmax(tl, dim=-1), 1e-4)


def test_permute_unpermute():
    torch.manual_seed(3)
    T, H, E, k = 300, 512, 8, 2
    x = torch.randn(T, H, device="cuda").bfloat16()
    logits = torch.randn(T, E, device="cuda")
    ti, tp = router.topk_softmax(logits, k)
    plan = router.build_padded_plan(ti, tp, E, router.expert_capacity(T, k, E, 1.0))
    perm = permute.permute_rows(x, plan.sorted_indices)
    assert torch.equal(perm, x[plan.sorted_indices])
    res = torch.randn(T, H, device="cuda").bfloat16()
    out = permute.unpermute_reduce(perm, plan.slot_of_token, res)
    ref = permute.unpermute_reduce(perm.cpu().float(), plan.slot_of_token.cpu(), res.cpu().float())
    _close(out, ref)


def test_fused_adam():
    from fluidmoe_b200.ops.optim import FusedAdam
    torch.manual_seed(4)
    p = torch.nn.Parameter(torch.randn(1000, 33, device="cuda").bfloat16())
    ref = torch.nn.Parameter(p.detach().float().clone())
    opt = FusedAdam([p], lr=1e-2, weight_decay=0.01, master_weights=True)
    ropt = torch.optim.AdamW([ref], lr=1e-2, weight_decay=0.01, eps=1e-8)
    for _ in range(3):
        g = torch.randn_like(ref)
        p.main_grad = g.clone()
        p._ar_buf_written = True
        ref.grad = g
        opt.step()
        ropt.step()
    _close(p, ref, 1e-2)


@pytest.mark.parametrize("T,E,k", [(512, 8, 2), (1000, 64, 6), (4096, 8, 2)])
def test_moe_plan_kernel_matches_prefix_sum_plan(T, E, k):
    torch.manual_seed(5)
    logits = torch.randn(T, E, device="cuda") + torch.linspace(0, 1.5, E, device="cuda")  # imbalance -> drops
    ti, tp = router.topk_softmax(logits, k)
    cap = router.expert_capacity(T, k, E, 1.0)
    got = router.build_padded_plan(ti, tp, E, cap)
    ref = router.build_padded_plan(ti.cpu(), tp.cpu(), E, cap)
    assert got.routing_map is None  # came from the CUDA kernel
    assert torch.equal(got.sorted_indices.cpu(), ref.sorted_indices)
    assert torch.equal(got.slot_of_token.cpu(), ref.slot_of_token)
    assert torch.equal(got.routed_per_expert.cpu(), ref.routed_per_expert)
    _close(got.permuted_probs, ref.permuted_probs, 1e-6)


def test_fused_cross_entropy():
    torch.manual_seed(6)
    T, V = 300, 32000
    logits = (torch.randn(T, V, device="cuda") * 3).bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[5] = -1
    ref_in = logits.float().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in, labels, ignore_index=-1, reduction="none")
    ref.sum().backward()
    work = logits.clone()
    loss = ew.cross_entropy_(work, labels, 1.0)
    _close(loss, ref, 1e-2)
    assert (work.float() - ref_in.grad).abs().max().item() < 1e-2


@pytest.mark.parametrize("aux,z", [(0.0, 0.0), (0.01, 0.001)])
def test_router_backward_kernel_matches_pytorch(aux, z, monkeypatch):
    from fluidmoe_b200 import _native
    T, E, k = 1000, 8, 2
    torch.manual_seed(3)
    logits = torch.randn(T, E, device="cuda")
    ti, tp = router.topk_softmax(logits, k)
    cap = router.expert_capacity(T, k, E, 1.0)
    plan = router.build_padded_plan(ti, tp, E, cap)
    dprobs = torch.randn(E * cap, device="cuda")
    tpe = plan.routed_per_expert.float()
    got = router.router_backward_logits(dprobs, plan, ti, tp, logits, E, aux, z, tpe, T)
    monkeypatch.setattr(_native, "use_native", lambda *a: False)
    ref = router.router_backward_logits(dprobs, plan, ti, tp, logits, E, aux, z, tpe, T)
    assert (got - ref).abs().max().item() < 1e-5 * max(1.0, ref.abs().max().item())


def test_adam_background_kernel_matches_fp32_reference():
    n = (1 << 20) + 4 * 37
    torch.manual_seed(7)
    p = (torch.randn(n, device="cuda") * 0.05).bfloat16()
    g = torch.randn(n, device="cuda")
    m = (torch.randn(n, device="cuda") * 0.1).bfloat16()
    v = (torch.rand(n, device="cuda") * 0.1).bfloat16()
    lr, b1, b2, eps, wd, step, gs = 1e-2, 0.9, 0.95, 1e-8, 0.1, 3, 0.5
    gf = g * gs
    m_ref = b1 * m.float() + (1 - b1) * gf
    v_ref = b2 * v.float() + (1 - b2) * gf * gf
    w = p.float()
    w_ref = w - lr * ((m_ref / (1 - b1 ** step)) / ((v_ref / (1 - b2 ** step)).sqrt() + eps) + wd * w)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    ew.adam_background(p, g, m, v, lr, b1, b2, eps, wd, step, grad_scale=gs, stream=side.cuda_stream)
    side.synchronize()
    for name, got, ref in (("m", m, m_ref), ("v", v, v_ref), ("p", p, w_ref)):
        err = ((got.float() - ref).norm() / ref.norm()).item()
        assert err < 6e-3, (name, err)


def test_symmetric_heap_canaries_detect_an_overrun(monkeypatch):
    """Debug guards of the symmetric heap: a write past the end of a buffer (simulated with an
    in-heap store, nothing faults) is reported with the allocation it belongs to."""
    from fluidmoe_b200.parallel.symm import SymmetricHeap
    monkeypatch.setenv("FLUIDMOE_SYMM_CANARY", "1")
    heap = SymmetricHeap(None, 1 << 20, torch.device("cuda", torch.cuda.current_device()))
    a = heap.alloc((1000,), torch.float32)
    b = heap.alloc((64, 8), torch.bfloat16)
    a.local.fill_(1.0)
    b.local.fill_(2.0)
    heap.check_canaries()                              # intact
    end_of_a = a.offset + 4096                         # 4000 bytes rounded up to the 1024-byte grain
    heap._slab[end_of_a + 7] = 0                       # one byte past the end of `a`
    with pytest.raises(RuntimeError, match="7 bytes past the end of allocation"):
        heap.check_canaries()
