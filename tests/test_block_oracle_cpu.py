"""The block's hand-written forward and backward against an independent autograd oracle
(``tests/oracle.py``: torch operators only, no library code), in one process and on two gloo ranks
(sequence- and expert-parallel), for LayerNorm / RMSNorm, GELU / SwiGLU, shared experts on and off,
and with the router's load-balancing and z losses on.
"""
import pytest
import torch

from tests import oracle
from tests.dist_utils import run_distributed

DIMS = dict(H=64, nh=4, nkv=2, F=96, E=4, k=2, s_loc=16, b=2)
# the anchor configuration: hidden 256, 8 heads x 32, 4 experts (2 per rank) 256 -> 512 -> 256 GELU, top-2,
# RMSNorm, RoPE, batch 2, 128 positions per rank, weights ~ N(0, 0.02)
CONFIG1 = dict(H=256, nh=8, nkv=8, F=512, E=4, k=2, s_loc=128, b=2, init_std=0.02)


def _layer_kwargs(norm_type, act, nsh, aux, cf, D=DIMS):
    return dict(dtype=torch.float32, device="cpu", router_dtype=torch.float32, activation_func=act,
                norm_type=norm_type, init_std=D.get("init_std", 0.2), capacity_factor=cf, num_shared_experts=nsh,
                aux_loss_coeff=1e-2 if aux else 0.0, z_loss_coeff=1e-3 if aux else 0.0,
                recompute_fc1=D.get("recompute_fc1", False))


def _build_full(norm_type, act, nsh, aux, cf, groups=(None, None), D=DIMS):
    from fluidmoe_b200.models.transformer import TransformerLayer
    torch.manual_seed(1)
    layer = TransformerLayer(D["H"], D["nh"], D["nkv"], D["F"], D["E"], D["k"], groups[0], groups[1],
                             **_layer_kwargs(norm_type, act, nsh, aux, cf, D))
    with torch.no_grad():   # norms away from identity so that their gradients are exercised
        g = torch.Generator().manual_seed(5)
        for n, p in layer.named_parameters():
            if n.startswith("ln"):
                p.add_(0.3 * torch.randn(p.shape, generator=g))
    return layer


def _inputs(world, D=DIMS):
    torch.manual_seed(2)
    S = world * D["s_loc"]
    return torch.randn(S, D["b"], D["H"]), torch.randn(S, D["b"], D["H"])


def _sharded_run(rank, world, norm_type, act, nsh, aux, cf, mode, sched_mode, D=DIMS):
    import torch.distributed as dist
    from fluidmoe_b200.distributed import init_parallel
    from fluidmoe_b200.models.transformer import TransformerLayer
    from fluidmoe_b200.ops.rope import make_rope_freqs
    from fluidmoe_b200.parallel.scheduler import get_backward_scheduler

    pc = init_parallel()
    solo = [dist.new_group([r]) for r in range(world)][rank]
    full = _build_full(norm_type, act, nsh, aux, cf, (solo, solo), D)
    layer = TransformerLayer(D["H"], D["nh"], D["nkv"], D["F"], D["E"], D["k"], pc.cp_group, pc.ep_group,
                             comm_mode=mode, moe_combine_chunks=2, moe_dispatch_chunks=2, attn_proj_chunks=2,
                             attn_qkv_chunks=2, **_layer_kwargs(norm_type, act, nsh, aux, cf, D))
    nle = D["E"] // world
    with torch.no_grad():
        src = dict(full.named_parameters())
        for n, p in layer.named_parameters():
            p.copy_(src[n][rank * nle:(rank + 1) * nle] if n in ("moe_w1", "moe_w2") else src[n])
    x_full, g_full = _inputs(world, D)
    rot = make_rope_freqs(world * D["s_loc"], D["H"] // D["nh"])
    if D.get("overhead"):
        from fluidmoe_b200.utils import overhead_profiler as op
        op.set_enabled(True)
        op.reset()
    sched = get_backward_scheduler()
    sched.configure_allreduce(sched_mode == "full", pc.dp_cp_group, pc.expert_dp_group,
                              gap_budgets={r: 1.0 for r in ("moe_combine", "moe_dispatch", "attn_proj", "attn_qkv")},
                              shared_ar_bw=1e6, expert_ar_bw=1e6)
    if sched_mode == "F":
        sched.disable()
    else:
        sched.enable(torch.device("cpu"))
        for key, val in D.get("sched_toggles", {}).items():
            assert hasattr(sched, key), key
            setattr(sched, key, val)
        expert = [layer.moe_w2, layer.moe_w1]
        sched.setup_ar_buffer([p for p in layer.parameters() if all(p is not e for e in expert)], True)
        sched.setup_expert_ar_buffer(expert, True)
    sl = slice(rank * D["s_loc"], (rank + 1) * D["s_loc"])
    x = x_full[sl].clone().requires_grad_(True)
    y = layer(x, rot)
    y.backward(g_full[sl])
    if sched_mode == "F":
        sched.sync_allreduce_params(list(layer.parameters()))
        grads = {n: p.grad.clone() for n, p in layer.named_parameters()}
    else:
        sched.finish_batch()
        grads = {n: p.main_grad.clone() for n, p in layer.named_parameters()}
    sched.clear_iteration()
    if D.get("overhead"):
        from fluidmoe_b200.utils import overhead_profiler as op
        buckets = op.summary_by_bucket()
        op.set_enabled(False)
        return y.detach(), x.grad, grads, buckets
    return y.detach(), x.grad, grads


def _oracle(world, norm_type, act, nsh, aux, cf, D=DIMS):
    from fluidmoe_b200.ops.rope import make_rope_freqs
    full = _build_full(norm_type, act, nsh, aux, cf, D=D)
    P = oracle.full_params_from_layers([full])
    x_full, g_full = _inputs(world, D)
    x = x_full.clone().requires_grad_(True)
    rot = make_rope_freqs(world * D["s_loc"], D["H"] // D["nh"])
    y, reg = oracle.block_forward(x, P, num_heads=D["nh"], num_kv_heads=D["nkv"], top_k=D["k"], world=world,
                                  activation=act, norm_type=norm_type, capacity_factor=cf, rotary=rot,
                                  aux_loss_coeff=1e-2 if aux else 0.0, z_loss_coeff=1e-3 if aux else 0.0)
    ((y * g_full).sum() + reg).backward()
    return y.detach(), x.grad, {n: p.grad for n, p in P.items()}


def _close(a, b, what, tol=2e-4):
    scale = b.abs().max().item() + 1e-9
    err = (a - b).abs().max().item() / scale
    assert err < tol, (what, err)


CASES = [("layernorm", "gelu", 0, False, 1.0), ("rmsnorm", "swiglu", 1, False, 1.0),
         ("rmsnorm", "gelu", 0, True, 1.0), ("layernorm", "swiglu", 1, True, 2.0),
         ("rmsnorm", "swiglu", 0, False, 0.0)]


@pytest.mark.parametrize("norm_type,act,nsh,aux,cf", CASES)
def test_block_matches_autograd_oracle_single_process(norm_type, act, nsh, aux, cf):
    from fluidmoe_b200.ops.rope import make_rope_freqs
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler, get_backward_scheduler
    BackwardScheduler.reset()
    get_backward_scheduler().disable()
    D = DIMS
    layer = _build_full(norm_type, act, nsh, aux, cf)
    x_full, g_full = _inputs(1)
    x = x_full.clone().requires_grad_(True)
    y = layer(x, make_rope_freqs(D["s_loc"], D["H"] // D["nh"]))
    y.backward(g_full)
    yo, dxo, go = _oracle(1, norm_type, act, nsh, aux, cf)
    _close(y.detach(), yo, "y")
    _close(x.grad, dxo, "dx")
    for n, p in layer.named_parameters():
        _close(p.grad, go[n], n)
    BackwardScheduler.reset()


@pytest.mark.parametrize("norm_type,act,nsh,aux,cf,mode,sched_mode", [
    ("layernorm", "gelu", 0, False, 1.0, "a2a", "F"),
    ("rmsnorm", "swiglu", 1, True, 1.0, "p2p", "full"),
    ("rmsnorm", "swiglu", 0, False, 0.0, "a2a", "FB"),
])
def test_block_matches_autograd_oracle_world2(norm_type, act, nsh, aux, cf, mode, sched_mode):
    """Sequence- and expert-parallel over two ranks.  Gradients come back averaged over the
    data-parallel group (pre-scale 1/world, then sum), so they are compared after scaling by the
    world size."""
    world = 2
    D = DIMS
    res = run_distributed(_sharded_run, world, norm_type, act, nsh, aux, cf, mode, sched_mode)
    yo, dxo, go = _oracle(world, norm_type, act, nsh, aux, cf)
    nle = D["E"] // world
    for r in range(world):
        y, dx, grads = res[r]
        sl = slice(r * D["s_loc"], (r + 1) * D["s_loc"])
        _close(y, yo[sl], f"y rank {r}")
        _close(dx, dxo[sl], f"dx rank {r}")
        for n, g in grads.items():
            ref = go[n][r * nle:(r + 1) * nle] if n in ("moe_w1", "moe_w2") else go[n]
            _close(g * world, ref, f"{n} rank {r}")


def test_anchor_configuration_world2_against_oracle():
    """The anchor configuration exactly as stated (fp32, gloo, EP = SP = 2): pairwise-overlap
    transport with the scheduler in full mode against the autograd oracle."""
    world, D = 2, CONFIG1
    res = run_distributed(_sharded_run, world, "rmsnorm", "gelu", 0, False, 1.0, "p2p", "full", D)
    yo, dxo, go = _oracle(world, "rmsnorm", "gelu", 0, False, 1.0, D)
    nle = D["E"] // world
    for r in range(world):
        y, dx, grads = res[r]
        sl = slice(r * D["s_loc"], (r + 1) * D["s_loc"])
        _close(y, yo[sl], f"y rank {r}")
        _close(dx, dxo[sl], f"dx rank {r}")
        for n, g in grads.items():
            ref = go[n][r * nle:(r + 1) * nle] if n in ("moe_w1", "moe_w2") else go[n]
            _close(g * world, ref, f"{n} rank {r}", tol=5e-4)


@pytest.mark.parametrize("half", ["attention", "moe"])
def test_single_half_layer_matches_full_layer_with_the_other_half_silenced(half):
    """``has_moe=False`` / ``has_attention=False`` must equal the full block whose other half
    contributes nothing (its output weights set to zero), in output, ``dx`` and the gradients of
    the active half; with a router logit prior on."""
    from fluidmoe_b200.models.transformer import TransformerLayer
    from fluidmoe_b200.ops.rope import make_rope_freqs
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler, get_backward_scheduler
    BackwardScheduler.reset()
    get_backward_scheduler().disable()
    D = DIMS
    kw = _layer_kwargs("rmsnorm", "swiglu", 1, False, 1.0)
    full = _build_full("rmsnorm", "swiglu", 1, False, 1.0)
    torch.manual_seed(1)
    part = TransformerLayer(D["H"], D["nh"], D["nkv"], D["F"], D["E"], D["k"], None, None,
                            has_attention=half == "attention", has_moe=half == "moe", **kw)
    part.load_state_dict(full.state_dict())
    bias = torch.log(1.0 / torch.arange(1, D["E"] + 1, dtype=torch.float32) ** 1.1)
    full.set_router_bias(bias)
    part.set_router_bias(bias)
    with torch.no_grad():
        if half == "attention":
            full.moe_w2.zero_()
            full.shared_w2.zero_()
        else:
            full.proj_weight.zero_()
    x_full, g_full = _inputs(1)
    rot = make_rope_freqs(D["s_loc"], D["H"] // D["nh"])
    outs = []
    for layer in (full, part):
        x = x_full.clone().requires_grad_(True)
        y = layer(x, rot)
        y.backward(g_full)
        outs.append((y.detach(), x.grad, {n: p.grad for n, p in layer.named_parameters()}))
    (yf, dxf, gf), (yp, dxp, gp) = outs
    _close(yp, yf, "y", 1e-5)
    _close(dxp, dxf, "dx", 1e-5)
    active = (("ln1_weight", "qkv_weight", "proj_weight") if half == "attention" else
              ("ln2_weight", "router_weight", "moe_w1", "moe_w2", "shared_w1", "shared_w2"))
    for n in active:
        _close(gp[n], gf[n], n, 1e-5)
    idle = ("ln2_weight", "router_weight", "moe_w1") if half == "attention" else ("ln1_weight", "qkv_weight")
    for n in idle:
        assert gp[n] is None or float(gp[n].abs().max()) == 0.0, n
    BackwardScheduler.reset()


@pytest.mark.parametrize("act,cf,world,mode", [("swiglu", 1.0, 1, "a2a"), ("gelu", 0.0, 1, "a2a"),
                                               ("swiglu", 1.0, 2, "p2p"), ("gelu", 0.0, 2, "a2a")])
def test_fc1_recompute_gives_the_same_gradients(act, cf, world, mode):
    """With ``recompute_fc1`` the FC1 pre-activation is not saved; the backward pass rebuilds it
    from the saved tokens and must still match the oracle (padded and dropless routing)."""
    D = dict(DIMS, recompute_fc1=True)
    if world == 1:
        from fluidmoe_b200.ops.rope import make_rope_freqs
        from fluidmoe_b200.parallel.scheduler import BackwardScheduler, get_backward_scheduler
        BackwardScheduler.reset()
        get_backward_scheduler().disable()
        layer = _build_full("rmsnorm", act, 0, False, cf, D=D)
        assert layer.recompute_fc1
        x_full, g_full = _inputs(1)
        x = x_full.clone().requires_grad_(True)
        y = layer(x, make_rope_freqs(D["s_loc"], D["H"] // D["nh"]))
        y.backward(g_full)
        results = [(y.detach(), x.grad, {n: p.grad for n, p in layer.named_parameters()})]
        BackwardScheduler.reset()
    else:
        results = run_distributed(_sharded_run, world, "rmsnorm", act, 0, False, cf, mode, "full", D)
    yo, dxo, go = _oracle(world, "rmsnorm", act, 0, False, cf)
    nle = DIMS["E"] // world
    for r, (y, dx, grads) in enumerate(results):
        sl = slice(r * DIMS["s_loc"], (r + 1) * DIMS["s_loc"])
        _close(y, yo[sl], "y")
        _close(dx, dxo[sl], "dx")
        for n, g in grads.items():
            ref = go[n][r * nle:(r + 1) * nle] if n in ("moe_w1", "moe_w2") else go[n]
            _close(g * world, ref, n)


@pytest.mark.parametrize("toggles", [
    dict(stage2_enabled=False),                          # weight gradients only at the end of backward
    dict(cross_region_flow=False),                       # every region drains its own queue
    dict(use_profiled_gaps=False),                       # no gap model: reductions wait for finish_batch
    dict(fixed_ar_budget=4096),                          # a fixed number of bytes per gap
    dict(pending_ar_enabled=False),                      # no trickled reductions after the exchanges
    dict(stage2_enabled=False, pending_ar_enabled=False, cross_region_flow=False),
    dict(skip_all_dw=True),                              # FLUID_SKIP_ALL_DW: no deferrable dW in any window
    dict(skip_dispatch_dw=True),                         # FLUID_SKIP_DISPATCH_DW: none in the dispatch-gradient window
])
def test_scheduler_ablation_switches_keep_the_gradients(toggles):
    """The switches the reference's ablation runs flip (tests/run_block_benchmark.py:286-323: stage-2
    weight gradients, cross-region flow, profiled gaps, fixed reduction budget, trickled
    reductions) change when work is submitted, never what is computed."""
    world = 2
    D = dict(DIMS, sched_toggles=toggles, overhead=True)
    res = run_distributed(_sharded_run, world, "rmsnorm", "swiglu", 1, False, 1.0, "p2p", "full", D)
    yo, dxo, go = _oracle(world, "rmsnorm", "swiglu", 1, False, 1.0)
    nle = DIMS["E"] // world
    for r in range(world):
        y, dx, grads, buckets = res[r]
        sl = slice(r * DIMS["s_loc"], (r + 1) * DIMS["s_loc"])
        _close(y, yo[sl], f"y rank {r}")
        _close(dx, dxo[sl], f"dx rank {r}")
        for n, g in grads.items():
            ref = go[n][r * nle:(r + 1) * nle] if n in ("moe_w1", "moe_w2") else go[n]
            _close(g * world, ref, f"{n} rank {r} {toggles}")
        # the host-overhead buckets of the scheduler were filled while it ran
        assert any(v > 0 for v in buckets.values()), buckets
