"""The whole block on one GPU (bf16, native kernels) against the CPU fp32 path of the same code."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("norm_type,act,nsh,E,k", [("layernorm", "gelu", 0, 4, 4), ("rmsnorm", "swiglu", 1, 4, 4),
                                                   ("rmsnorm", "swiglu", 0, 8, 2)])
def test_layer_forward_backward_matches_cpu(norm_type, act, nsh, E, k):
    """With k == E every expert is selected and nothing is dropped, so the block is a continuous
    function of its inputs and bf16 results must track the fp32 path closely.  With k < E a few
    tokens whose logits nearly tie pick other experts in bf16; that case only checks that almost
    all positions agree."""
    from fluidmoe_b200.models.transformer import TransformerLayer
    from fluidmoe_b200.ops.rope import make_rope_freqs
    from fluidmoe_b200.ops import gemm
    from fluidmoe_b200.parallel.scheduler import get_backward_scheduler

    get_backward_scheduler().disable()
    torch.manual_seed(0)
    H, nh, nkv, F = 512, 8, 4, 768
    s, b = 256, 2
    kw = dict(router_dtype=torch.float32, activation_func=act, norm_type=norm_type,
              num_shared_experts=nsh, init_std=0.05)
    cpu = TransformerLayer(H, nh, nkv, F, E, k, None, None, dtype=torch.float32, device="cpu", **kw)
    with torch.no_grad():
        for p in cpu.parameters():
            p.copy_(p.bfloat16().float())
    gpu = TransformerLayer(H, nh, nkv, F, E, k, None, None, dtype=torch.bfloat16, device="cuda", **kw)
    gpu.load_state_dict({n: v.bfloat16() for n, v in cpu.state_dict().items()})
    x = torch.randn(s, b, H).bfloat16().float()
    g = torch.randn(s, b, H).bfloat16().float()
    rot = make_rope_freqs(s, 32)
    xc = x.clone().requires_grad_(True)
    yc = cpu(xc, rot)
    yc.backward(g)
    xg = x.cuda().bfloat16().requires_grad_(True)
    yg = gpu(xg, rot.cuda())
    yg.backward(g.cuda().bfloat16())
    torch.cuda.synchronize()
    gemm.check_status()

    # Routing is discrete: a token whose k-th and (k+1)-th logits nearly tie may pick another
    # expert in bf16 than in fp32.  Judge by the fraction of positions that agree and by the
    # relative Frobenius error, not by the single worst element.
    def fro(a, b_):
        a, b_ = a.float().cpu(), b_.float()
        return ((a - b_).norm() / (b_.norm() + 1e-9)).item()

    tok_err = (yg.float().cpu() - yc).abs().amax(-1) / (yc.abs().amax(-1) + 1e-6)
    assert (tok_err < 5e-2).float().mean().item() > 0.97, (tok_err < 5e-2).float().mean().item()
    if k < E:
        return
    assert fro(yg, yc) < 5e-2, fro(yg, yc)
    assert fro(xg.grad, xc.grad) < 8e-2, fro(xg.grad, xc.grad)
    for (n, pg), (_, pc) in zip(gpu.named_parameters(), cpu.named_parameters()):
        assert fro(pg.grad, pc.grad) < 8e-2, (n, fro(pg.grad, pc.grad))


def test_dropless_fine_grained_layer_runs_and_matches_cpu():
    """Fine-grained MoE: many small experts, top-6, shared experts, skewed routing, no dropping."""
    from fluidmoe_b200.models.transformer import TransformerLayer
    from fluidmoe_b200.ops import gemm
    from fluidmoe_b200.parallel.scheduler import get_backward_scheduler

    get_backward_scheduler().disable()
    torch.manual_seed(0)
    H, nh, nkv, F, E, k = 512, 4, 4, 256, 16, 16       # k == E keeps the comparison continuous
    s, b = 128, 2
    kw = dict(router_dtype=torch.float32, activation_func="swiglu", norm_type="rmsnorm",
              num_shared_experts=2, init_std=0.05, capacity_factor=0.0)
    cpu = TransformerLayer(H, nh, nkv, F, E, k, None, None, dtype=torch.float32, device="cpu", **kw)
    with torch.no_grad():
        for p in cpu.parameters():
            p.copy_(p.bfloat16().float())
    gpu = TransformerLayer(H, nh, nkv, F, E, k, None, None, dtype=torch.bfloat16, device="cuda", **kw)
    gpu.load_state_dict({n: v.bfloat16() for n, v in cpu.state_dict().items()})
    x = torch.randn(s, b, H).bfloat16().float()
    g = torch.randn(s, b, H).bfloat16().float()
    xc = x.clone().requires_grad_(True)
    yc = cpu(xc)
    yc.backward(g)
    xg = x.cuda().bfloat16().requires_grad_(True)
    yg = gpu(xg)
    yg.backward(g.cuda().bfloat16())
    torch.cuda.synchronize()
    gemm.check_status()

    def fro(a, b_):
        a, b_ = a.float().cpu(), b_.float()
        return ((a - b_).norm() / (b_.norm() + 1e-9)).item()
    assert fro(yg, yc) < 5e-2
    assert fro(xg.grad, xc.grad) < 8e-2
    for (n, pg), (_, pc) in zip(gpu.named_parameters(), cpu.named_parameters()):
        assert fro(pg.grad, pc.grad) < 8e-2, n
