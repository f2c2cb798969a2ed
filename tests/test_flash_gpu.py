"""tcgen05 flash attention (forward) against an fp32 reference."""
import math

import pytest
import torch

from fluidmoe_b200.ops import attention, flash, gemm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("version", [1, 2])
@pytest.mark.parametrize("s,b,G,qpg", [(128, 1, 1, 1), (256, 2, 2, 4), (1000, 1, 1, 4), (2048, 1, 2, 2), (640, 1, 1, 2)])
def test_flash_fwd_matches_reference(s, b, G, qpg, version):
    d = 128
    torch.manual_seed(0)
    qkv = torch.randn(s, b, G, (qpg + 2) * d, device="cuda").bfloat16()
    assert flash.supported(qkv, d)
    out, lse = flash.flash_attn_fwd_packed(qkv, qpg, d, 1.0 / math.sqrt(d), version)
    torch.cuda.synchronize()
    gemm.check_status()
    heads = qkv.float().cpu().view(s, b, G, qpg + 2, d)
    q = heads[:, :, :, :qpg].reshape(s, b, G * qpg, d)
    ro, rl = attention.attention_fwd(q, heads[:, :, :, qpg], heads[:, :, :, qpg + 1], 1.0 / math.sqrt(d), True)
    err = (out.float().cpu() - ro).abs().max().item()
    assert err < 3e-2, err
    assert (lse.cpu() - rl).abs().max().item() < 2e-2


@pytest.mark.parametrize("version", [1, 2])
def test_flash_fwd_speed(version):
    s, b, G, qpg, d = 8192, 1, 2, 4, 128
    qkv = torch.randn(s, b, G, (qpg + 2) * d, device="cuda").bfloat16()
    for _ in range(3):
        flash.flash_attn_fwd_packed(qkv, qpg, d, 0.088, version)
    torch.cuda.synchronize()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for _ in range(10):
        flash.flash_attn_fwd_packed(qkv, qpg, d, 0.088, version)
    en.record()
    torch.cuda.synchronize()
    gemm.check_status()
    ms = st.elapsed_time(en) / 10
    flops = 4 * s * s * G * qpg * d / 2
    print(f"\nflash fwd v{version} s={s} heads={G*qpg}: {ms:.3f} ms, {flops / ms / 1e9:.1f} TFLOP/s")


@pytest.mark.parametrize("fwd", ["native", "library"])
def test_attention_backward_from_saved_output(fwd):
    """Backward from the saved output and log-sum-exp (no forward recompute) against fp32."""
    s, b, G, qpg, d = 512, 1, 2, 2, 128
    torch.manual_seed(1)
    qkv = torch.randn(s, b, G, (qpg + 2) * d, device="cuda").bfloat16()
    heads = qkv.view(s, b, G, qpg + 2, d)
    q = heads[:, :, :, :qpg].reshape(s, b, G * qpg, d)
    k, v = heads[:, :, :, qpg], heads[:, :, :, qpg + 1]
    scale = 1.0 / math.sqrt(d)
    if fwd == "native":
        out, lse = flash.flash_attn_fwd_packed(qkv, qpg, d, scale)
    else:
        out, lse = attention._sdpa_fwd(q, k, v, scale, True)
    dout = torch.randn_like(out)
    dq, dk, dv = attention.attention_bwd(dout, q, k, v, out, lse, scale, True)
    torch.cuda.synchronize()
    qc, kc, vc = (t.float().cpu() for t in (q, k, v))
    ro, rl = attention.attention_fwd(qc, kc, vc, scale, True)
    rdq, rdk, rdv = attention.attention_bwd(dout.float().cpu(), qc, kc, vc, ro, rl, scale, True)
    for got, ref in ((dq, rdq), (dk, rdk), (dv, rdv)):
        err = (got.float().cpu() - ref).norm() / ref.norm()
        assert err < 3e-2, err


@pytest.mark.parametrize("version,head_split", [(1, None), (2, False), (2, 2), (2, None)])
@pytest.mark.parametrize("s,b,G,qpg", [(256, 1, 1, 1), (512, 1, 2, 2), (1000, 2, 1, 4)])
def test_flash_bwd_native_matches_reference(s, b, G, qpg, version, head_split):
    if head_split == 2 and qpg % 2:
        pytest.skip("query heads per group not divisible")
    d = 128
    torch.manual_seed(2)
    qkv = torch.randn(s, b, G, (qpg + 2) * d, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(d)
    out, lse = flash.flash_attn_fwd_packed(qkv, qpg, d, scale)
    dout = torch.randn_like(out)
    dqkv = flash.flash_attn_bwd_packed(dout, qkv, out, lse, qpg, d, scale, version=version, head_split=head_split)
    torch.cuda.synchronize()
    gemm.check_status()
    heads = qkv.float().cpu().view(s, b, G, qpg + 2, d)
    q = heads[:, :, :, :qpg].reshape(s, b, G * qpg, d)
    k, v = heads[:, :, :, qpg], heads[:, :, :, qpg + 1]
    ro, rl = attention.attention_fwd(q, k, v, scale, True)
    rdq, rdk, rdv = attention.attention_bwd(dout.float().cpu(), q, k, v, ro, rl, scale, True)
    got = dqkv.float().cpu().view(s, b, G, qpg + 2, d)
    for name, g_, r_ in (("dq", got[:, :, :, :qpg].reshape(s, b, G * qpg, d), rdq), ("dk", got[:, :, :, qpg], rdk),
                         ("dv", got[:, :, :, qpg + 1], rdv)):
        err = ((g_ - r_).norm() / r_.norm()).item()
        assert err < 3e-2, (name, err)


@pytest.mark.parametrize("version", [1, 2])
def test_flash_bwd_speed(version):
    s, b, G, qpg, d = 8192, 1, 2, 4, 128
    qkv = torch.randn(s, b, G, (qpg + 2) * d, device="cuda").bfloat16()
    out, lse = flash.flash_attn_fwd_packed(qkv, qpg, d, 0.088)
    dout = torch.randn_like(out)
    for _ in range(2):
        flash.flash_attn_bwd_packed(dout, qkv, out, lse, qpg, d, 0.088, version=version)
    torch.cuda.synchronize()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for _ in range(5):
        flash.flash_attn_bwd_packed(dout, qkv, out, lse, qpg, d, 0.088, version=version)
    en.record()
    torch.cuda.synchronize()
    gemm.check_status()
    ms = st.elapsed_time(en) / 5
    flops = 2.5 * 4 * s * s * G * qpg * d / 2
    print(f"\nflash bwd v{version} s={s} heads={G*qpg}: {ms:.3f} ms, {flops / ms / 1e9:.1f} TFLOP/s")
