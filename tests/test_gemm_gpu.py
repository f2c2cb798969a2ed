"""tcgen05 GEMM against a PyTorch fp32 reference of the same op."""
import pytest
import torch

from fluidmoe_b200.ops import gemm

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _close(got, ref, tol=2e-2):
    got, ref = got.float(), ref.float()
    err = (got - ref).abs().max().item()
    denom = ref.abs().max().item() + 1e-6
    assert err / denom < tol, f"max err {err} vs scale {denom}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 128), (256, 512, 256), (300, 520, 192), (1024, 1024, 1024), (77, 72, 72)])
@pytest.mark.parametrize("layout", ["nk", "kn"])
def test_dense(M, N, K, layout):
    torch.manual_seed(0)
    a = _rand(M, K)
    w = _rand(N, K) if layout == "nk" else _rand(K, N)
    out = gemm.grouped_gemm(a, w, b_layout=layout)
    torch.cuda.synchronize()
    gemm.check_status()
    ref = a.float() @ (w.float().t() if layout == "nk" else w.float())
    _close(out, ref)


def test_dense_fp32_accumulate():
    a, w = _rand(256, 128), _rand(384, 128)
    out = torch.ones(256, 384, device="cuda", dtype=torch.float32)
    gemm.grouped_gemm(a, w, b_layout="nk", out=out, accumulate=True, alpha=0.5)
    torch.cuda.synchronize()
    gemm.check_status()
    _close(out, 1.0 + 0.5 * (a.float() @ w.float().t()))


@pytest.mark.parametrize("layout", ["nk", "kn"])
def test_grouped_variable_rows(layout):
    torch.manual_seed(1)
    G, K, N = 4, 128, 320
    rows = torch.tensor([130, 0, 64, 257], dtype=torch.int32)
    offs = torch.tensor([0, 192, 192, 256], dtype=torch.int32)
    total = 256 + 320
    a = _rand(total, K)
    w = _rand(G, N, K) if layout == "nk" else _rand(G, K, N)
    out = gemm.grouped_gemm(a, w, b_layout=layout, group_rows=rows.cuda(), group_offs=offs.cuda())
    torch.cuda.synchronize()
    gemm.check_status()
    for g in range(G):
        o, r = offs[g].item(), rows[g].item()
        wg = w[g].float().t() if layout == "nk" else w[g].float()
        _close(out[o:o + r], a[o:o + r].float() @ wg) if r else None


@pytest.mark.parametrize("act", ["gelu", "silu", "swiglu"])
def test_fc1_act_prob(act):
    torch.manual_seed(2)
    G, H, F, cap = 2, 256, 384, 192
    a = _rand(G * cap, H)
    w = _rand(G, H, 2 * F if act == "swiglu" else F, scale=0.05)
    probs = torch.rand(G * cap, device="cuda")
    out, pre = gemm.grouped_gemm_act(a, w, probs, activation=act, uniform_rows=cap)
    torch.cuda.synchronize()
    gemm.check_status()
    for g in range(G):
        x = a[g * cap:(g + 1) * cap].float() @ w[g].float()
        _close(pre[g * cap:(g + 1) * cap], x)
        ref = gemm.act_ref(x, act) * probs[g * cap:(g + 1) * cap, None]
        _close(out[g * cap:(g + 1) * cap], ref)


@pytest.mark.parametrize("act", ["gelu", "swiglu"])
def test_fc2_dx_dact(act):
    torch.manual_seed(3)
    G, H, F, cap = 2, 256, 384, 160
    dy = _rand(G * cap, H)
    w2 = _rand(G, F, H, scale=0.05)
    pre = _rand(G * cap, 2 * F if act == "swiglu" else F)
    probs = torch.rand(G * cap, device="cuda")
    dpre, dprobs = gemm.grouped_gemm_dact(dy, w2, pre, probs, activation=act, uniform_rows=cap)
    torch.cuda.synchronize()
    gemm.check_status()
    rdpre, rdprobs = gemm.grouped_gemm_dact(dy.cpu(), w2.cpu(), pre.cpu(), probs.cpu(), activation=act, uniform_rows=cap)
    _close(dpre.cpu(), rdpre)
    _close(dprobs.cpu(), rdprobs)


def test_wgrad_grouped():
    torch.manual_seed(4)
    G, M, N = 3, 256, 320
    rows = torch.tensor([128, 70, 200], dtype=torch.int32)
    offs = torch.tensor([0, 128, 256], dtype=torch.int32)
    total = 512
    a, dy = _rand(total, M), _rand(total, N)
    # rows outside the groups must be zero (64-row contraction blocks)
    mask = torch.zeros(total, dtype=torch.bool)
    for o, r in zip(offs.tolist(), rows.tolist()):
        mask[o:o + r] = True
    a[~mask.cuda()] = 0
    out = torch.full((G, M, N), 2.0, device="cuda")
    gemm.grouped_gemm_wgrad(a, dy, G, group_rows=rows.cuda(), group_offs=offs.cuda(), out=out, accumulate=True)
    torch.cuda.synchronize()
    gemm.check_status()
    for g in range(G):
        o, r = offs[g].item(), rows[g].item()
        _close(out[g], 2.0 + a[o:o + r].float().t() @ dy[o:o + r].float())


def test_large_perf_smoke():
    a, w = _rand(4096, 4096), _rand(4096, 4096)
    for _ in range(3):
        out = gemm.grouped_gemm(a, w, b_layout="nk")
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        out = gemm.grouped_gemm(a, w, b_layout="nk")
    e.record()
    torch.cuda.synchronize()
    gemm.check_status()
    ms = s.elapsed_time(e) / 10
    print(f"\n4096^3 bf16: {ms:.3f} ms, {2 * 4096**3 / ms / 1e9:.1f} TFLOP/s")
    _close(out, a.float() @ w.float().t())


@pytest.fixture
def cta_pair():
    old = gemm.CTA_PAIR
    gemm.CTA_PAIR = 1
    yield
    gemm.CTA_PAIR = old


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 256), (300, 520, 192), (1024, 1024, 1024)])
@pytest.mark.parametrize("layout", ["nk", "kn"])
def test_cta_pair_dense(cta_pair, M, N, K, layout):
    torch.manual_seed(0)
    a = _rand(M, K)
    w = _rand(N, K) if layout == "nk" else _rand(K, N)
    out = gemm.grouped_gemm(a, w, b_layout=layout)
    torch.cuda.synchronize()
    gemm.check_status()
    _close(out, a.float() @ (w.float().t() if layout == "nk" else w.float()))


def test_cta_pair_grouped_fused_epilogues(cta_pair):
    torch.manual_seed(2)
    G, H, F, cap = 2, 256, 384, 320
    a = _rand(G * cap, H)
    w = _rand(G, H, 2 * F, scale=0.05)
    probs = torch.rand(G * cap, device="cuda")
    out, pre = gemm.grouped_gemm_act(a, w, probs, activation="swiglu", uniform_rows=cap)
    dy = _rand(G * cap, H)
    w2 = _rand(G, F, H, scale=0.05)
    dpre, dprobs = gemm.grouped_gemm_dact(dy, w2, pre, probs, activation="swiglu", uniform_rows=cap)
    g1 = gemm.grouped_gemm_wgrad(a, dpre, G, uniform_rows=cap)
    torch.cuda.synchronize()
    gemm.check_status()
    for g in range(G):
        x = a[g * cap:(g + 1) * cap].float() @ w[g].float()
        _close(pre[g * cap:(g + 1) * cap], x)
        _close(out[g * cap:(g + 1) * cap], gemm.act_ref(x, "swiglu") * probs[g * cap:(g + 1) * cap, None])
        _close(g1[g], a[g * cap:(g + 1) * cap].float().t() @ dpre[g * cap:(g + 1) * cap].float())
    rdpre, rdprobs = gemm.grouped_gemm_dact(dy.cpu(), w2.cpu(), pre.cpu(), probs.cpu(), activation="swiglu", uniform_rows=cap)
    _close(dpre.cpu(), rdpre)
    _close(dprobs.cpu(), rdprobs)


def test_cta_pair_speed(cta_pair):
    a, w = _rand(8192, 8192), _rand(8192, 8192)
    for _ in range(3):
        out = gemm.grouped_gemm(a, w, b_layout="nk")
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        out = gemm.grouped_gemm(a, w, b_layout="nk")
    e.record()
    torch.cuda.synchronize()
    gemm.check_status()
    ms = s.elapsed_time(e) / 10
    print(f"\n8192^3 bf16 (CTA pair): {ms:.3f} ms, {2 * 8192**3 / ms / 1e9:.1f} TFLOP/s")


@pytest.mark.parametrize("cta_pair", [0, 1])
@pytest.mark.parametrize("G,rows_per,M,N", [(2, 256, 256, 512), (3, 128, 384, 264)])
def test_wgrad_adam_epilogue_matches_fp32_reference(G, rows_per, M, N, cta_pair, monkeypatch):
    """Optimizer in the weight-gradient epilogue == fp32 gradient followed by an fp32 AdamW update
    (the PyTorch reference of the same op), up to the bf16 rounding of parameter and moments."""
    monkeypatch.setattr(gemm, "CTA_PAIR", cta_pair)
    torch.manual_seed(5)
    a = torch.randn(G * rows_per, M, device="cuda").bfloat16()
    dy = torch.randn(G * rows_per, N, device="cuda").bfloat16()
    p = (torch.randn(G, M, N, device="cuda") * 0.05).bfloat16()
    m = (torch.randn(G, M, N, device="cuda") * 0.1).bfloat16()
    v = (torch.rand(G, M, N, device="cuda") * 0.1).bfloat16()
    lr, b1, b2, eps, wd, step, gs = 1e-2, 0.9, 0.95, 1e-8, 0.1, 3, 0.25
    g = torch.stack([a[i * rows_per:(i + 1) * rows_per].float().t() @ dy[i * rows_per:(i + 1) * rows_per].float()
                     for i in range(G)]) * gs
    m_ref = b1 * m.float() + (1 - b1) * g
    v_ref = b2 * v.float() + (1 - b2) * g * g
    w = p.float()
    w_ref = w - lr * ((m_ref / (1 - b1 ** step)) / ((v_ref / (1 - b2 ** step)).sqrt() + eps) + wd * w)
    gemm.grouped_gemm_wgrad_adam(a, dy, G, p, m, v, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd,
                                 step=step, grad_scale=gs, uniform_rows=rows_per)
    torch.cuda.synchronize()
    gemm.check_status()
    for name, got, ref in (("m", m, m_ref), ("v", v, v_ref), ("p", p, w_ref)):
        err = ((got.float() - ref).norm() / ref.norm()).item()
        assert err < 6e-3, (name, err)


def test_cta_pair_claimed_tile_order_few_pairs_many_launches(cta_pair):
    """Two CTA pairs claim the 64 tiles of the problem one by one (the order is dynamic whenever
    there are more tiles than pairs); 80 launches walk the claim counters round more than once,
    and a second stream, with a workspace of its own, runs beside the first."""
    torch.manual_seed(3)
    a = _rand(2048, 256)
    w = _rand(2048, 256)
    ref = a.float() @ w.float().t()
    side = torch.cuda.Stream()
    outs = []
    for i in range(80):
        outs.append(gemm.grouped_gemm(a, w, b_layout="nk", max_ctas=4))
        if i % 8 == 0:
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                outs.append(gemm.grouped_gemm(a, w, b_layout="nk", max_ctas=6))
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    gemm.check_status()
    for o in (outs[0], outs[1], outs[40], outs[-1]):
        _close(o, ref)
    assert all(torch.equal(o, outs[0]) for o in outs[1:])


def test_cta_pair_claimed_tile_order_with_row_counts_on_the_device(cta_pair):
    """Row counts in device memory: the host only knows a bound of the tile count, pairs stop at
    the first claim past the last tile, and empty groups contribute no tile."""
    torch.manual_seed(4)
    G, K, N = 6, 128, 1024
    rows = torch.tensor([700, 0, 256, 1, 1030, 0], dtype=torch.int32)
    offs = torch.tensor([0, 768, 768, 1024, 1280, 2560], dtype=torch.int32)
    a = _rand(2560, K)
    w = _rand(G, N, K)
    out = gemm.grouped_gemm(a, w, b_layout="nk", group_rows=rows.cuda(), group_offs=offs.cuda(), max_ctas=4)
    torch.cuda.synchronize()
    gemm.check_status()
    for g in range(G):
        o, r = offs[g].item(), rows[g].item()
        if r:
            _close(out[o:o + r], a[o:o + r].float() @ w[g].float().t())
