"""Multi-process CPU (gloo) checks: the overlapped layer against plain baselines.

One MoE transformer layer, fp32, world 2 (EP = SP = 2), hidden 256, 8 query / 4 KV heads x 32,
causal, RoPE, RMSNorm, 4 experts with FFN 512, GELU, top-2, batch 2, 32 positions per rank: every
transport and scheduler mode against the plain all-to-all path.  (The anchor configuration with
128 positions per rank and 8 x 32 heads is checked against an independent autograd oracle in
``test_block_oracle_cpu.py``.)
"""
import pytest
import torch

from tests.dist_utils import run_distributed


def _layer_vs_single(rank, world, mode, sched_mode, chunks, norm_type, act, capacity_factor=1.0, eager_ar=False):
    import torch.distributed as dist
    from fluidmoe_b200.distributed import init_parallel
    from fluidmoe_b200.models.transformer import TransformerLayer
    from fluidmoe_b200.ops.rope import make_rope_freqs
    from fluidmoe_b200.parallel.scheduler import get_backward_scheduler

    torch.manual_seed(0)
    H, nh, nkv, F, E, k = 256, 8, 4, 512, 4, 2
    s_loc, b = 32, 2
    pc = init_parallel()
    kw = dict(dtype=torch.float32, device="cpu", router_dtype=torch.float32, activation_func=act,
              norm_type=norm_type, init_std=0.05, capacity_factor=capacity_factor)
    # every rank builds the same full single-process layer, then its sharded twin
    torch.manual_seed(1)
    solo = [dist.new_group([r]) for r in range(world)][rank]   # a group of this rank alone
    ref = TransformerLayer(H, nh, nkv, F, E, k, solo, solo, **kw)
    layer = TransformerLayer(H, nh, nkv, F, E, k, pc.cp_group, pc.ep_group, comm_mode=mode,
                             moe_combine_chunks=chunks, moe_dispatch_chunks=chunks,
                             attn_proj_chunks=chunks, attn_qkv_chunks=chunks, **kw)
    nle = E // world
    with torch.no_grad():
        for n, p in layer.named_parameters():
            src = dict(ref.named_parameters())[n]
            if n in ("moe_w1", "moe_w2"):
                p.copy_(src[rank * nle:(rank + 1) * nle])
            else:
                p.copy_(src)
    torch.manual_seed(2)
    x_full = torch.randn(world * s_loc, b, H)
    g_full = torch.randn(world * s_loc, b, H)
    rot = make_rope_freqs(world * s_loc, 16)
    sched = get_backward_scheduler()
    sched.configure_allreduce(sched_mode == "full", pc.dp_cp_group, pc.expert_dp_group,
                              gap_budgets={r: 1.0 for r in ("moe_combine", "moe_dispatch", "attn_proj", "attn_qkv")},
                              shared_ar_bw=1e6, expert_ar_bw=1e6)
    sched.eager_ar = bool(eager_ar)
    sched.eager_ar_min_bytes = 0
    if sched_mode == "F":
        sched.disable()
    else:
        sched.enable(torch.device("cpu"))
        expert = [layer.moe_w2, layer.moe_w1]
        shared = [p for p in layer.parameters() if all(p is not e for e in expert)]
        sched.setup_ar_buffer(shared, accumulate_in_fp32=True)
        sched.setup_expert_ar_buffer(expert, accumulate_in_fp32=True)
    x = x_full[rank * s_loc:(rank + 1) * s_loc].clone().requires_grad_(True)
    y = layer(x, rot)
    y.backward(g_full[rank * s_loc:(rank + 1) * s_loc])
    if sched_mode == "F":
        sched.sync_allreduce_params(list(layer.parameters()))
        grads = {n: p.grad for n, p in layer.named_parameters()}
    else:
        sched.finish_batch()
        grads = {n: p.main_grad.clone() for n, p in layer.named_parameters()}
        stats = sched.get_stats()
        assert stats["pending_dw_at_finish"] == 0 and stats["completed_dw_tasks"] == stats["total_dw_tasks"]
    sched.clear_iteration()
    return (y.detach(), x.grad, grads)


@pytest.mark.parametrize("mode,sched_mode,chunks", [("p2p", "F", 1), ("p2p", "FB", 2), ("a2a", "full", 4), ("p2p", "full", 2)])
def test_overlap_matches_baseline_world2(mode, sched_mode, chunks):
    """Every transport / scheduler mode must produce the outputs and gradients of the plain
    all-to-all path with the scheduler off."""
    base = run_distributed(_layer_vs_single, 2, "a2a", "F", 1, "rmsnorm", "gelu")
    got = run_distributed(_layer_vs_single, 2, mode, sched_mode, chunks, "rmsnorm", "gelu")
    for r in range(2):
        yb, gxb, gb = base[r]
        y, gx, g = got[r]
        assert torch.allclose(y, yb, atol=2e-5), (y - yb).abs().max()
        assert torch.allclose(gx, gxb, atol=2e-4), (gx - gxb).abs().max()
        for n in gb:
            scale = gb[n].abs().max().item() + 1e-6
            assert (g[n] - gb[n]).abs().max().item() / scale < 1e-4, n


def test_eager_allreduce_matches_baseline_world2():
    """Gradient reduction started right after each batch of weight-gradient tasks (the policy used
    with the device-initiated transports) gives the same gradients as the reduction at the end."""
    base = run_distributed(_layer_vs_single, 2, "a2a", "F", 1, "rmsnorm", "gelu")
    got = run_distributed(_layer_vs_single, 2, "p2p", "full", 2, "rmsnorm", "gelu", 1.0, True)
    for r in range(2):
        yb, gxb, gb = base[r]
        y, gx, g = got[r]
        assert torch.allclose(y, yb, atol=2e-5)
        for n in gb:
            scale = gb[n].abs().max().item() + 1e-6
            assert (g[n] - gb[n]).abs().max().item() / scale < 1e-4, n


def _moe_vs_moebaseline(rank, world):
    """Hand-written MoE forward/backward (p2p overlap transport) against MoEBaseline autograd."""
    from fluidmoe_b200.distributed import init_parallel
    from fluidmoe_b200.models import moe
    from fluidmoe_b200.ops import permute
    from fluidmoe_b200.parallel.schedule import MultiCardOverlapContext
    from fluidmoe_b200.parallel.scheduler import get_backward_scheduler

    pc = init_parallel()
    H, F, E, k, T = 256, 512, 4, 2, 256
    torch.manual_seed(10 + rank)
    x = torch.randn(T, H, requires_grad=True)
    g = torch.randn(T, H)
    torch.manual_seed(3)
    base = moe.MoEBaseline(H, F, E, k, pc.ep_group, activation="gelu", dtype=torch.float32, device="cpu", init_std=0.05)
    with torch.no_grad():  # all ranks drew the same full-size weights; keep this rank's experts
        pass
    y_ref = base(x)
    y_ref.backward(g)
    ref = dict(y=y_ref.detach(), dx=x.grad.clone(), dw1=base.moe_w1.grad.clone(), dw2=base.moe_w2.grad.clone(),
               dr=base.router_weight.grad.clone())
    # hand-written path
    sched = get_backward_scheduler()
    sched.disable()
    ctx = MultiCardOverlapContext(torch.device("cpu"), world, world)
    plan = moe.EPPlan(T, H, E, k, pc.ep_group, 1.0, torch.float32, "cpu", ctx)
    xd = x.detach()
    (perm, probs, sidx, _, top_idx, top_probs, logits, _, rplan) = moe.router_forward(
        xd, base.router_weight, E, k, pc.ep_group, 1.0, plan, torch.float32)
    st = moe.dispatch_fc1_forward(plan, perm, probs, base.moe_w1.detach(), "gelu", "p2p")
    comb = moe.fc2_combine_forward(plan, st, base.moe_w2.detach(), "p2p")
    y = permute.unpermute_reduce(comb, rplan.slot_of_token)
    gperm = permute.permute_rows(g, rplan.sorted_indices)
    dfc2, dpre, dprobs = moe.combine_fc2_backward(plan, gperm, st, base.moe_w2.detach(), "gelu", 1, "a2a")
    from fluidmoe_b200.ops import gemm
    dw2 = gemm.grouped_gemm_wgrad(st.act_em, dfc2, plan.num_local_experts, uniform_rows=world * plan.expert_capacity)
    dw1 = gemm.grouped_gemm_wgrad(st.tokens_em, dpre, plan.num_local_experts, uniform_rows=world * plan.expert_capacity)
    dperm = moe.fc1_dispatch_backward(plan, dpre, base.moe_w1.detach(), 1, "a2a")
    from fluidmoe_b200.parallel import comm
    from fluidmoe_b200.ops import router as R
    dprobs_perm = comm.all_to_all(moe.expert_to_rank_major(dprobs, world, plan.num_local_experts, plan.expert_capacity).contiguous(), pc.ep_group)
    dlogits = R.router_backward_logits(dprobs_perm, rplan, top_idx, top_probs, logits, E)
    dx = permute.unpermute_reduce(dperm, rplan.slot_of_token) + dlogits @ base.router_weight.detach().t()
    dr = xd.t() @ dlogits
    out = {}
    for name, a, b_ in [("y", y, ref["y"]), ("dx", dx, ref["dx"]), ("dw1", dw1, ref["dw1"]), ("dw2", dw2, ref["dw2"]), ("dr", dr, ref["dr"])]:
        out[name] = ((a - b_).abs().max().item(), b_.abs().max().item())
    return out


def test_moe_overlap_matches_moebaseline_world2():
    for res in run_distributed(_moe_vs_moebaseline, 2):
        for name, (err, scale) in res.items():
            assert err / (scale + 1e-9) < 1e-4, (name, err, scale)


def test_dropless_matches_padded_without_drops_world2():
    """With capacity = all tokens nothing is dropped in padded mode, so the variable-split
    (dropless) path must give the same outputs and gradients."""
    base = run_distributed(_layer_vs_single, 2, "a2a", "F", 1, "rmsnorm", "swiglu", 2.0)   # E/k = 2 -> cap = T
    got = run_distributed(_layer_vs_single, 2, "a2a", "FB", 1, "rmsnorm", "swiglu", 0.0)
    for r in range(2):
        yb, gxb, gb = base[r]
        y, gx, g = got[r]
        assert torch.allclose(y, yb, atol=2e-5), (y - yb).abs().max()
        assert torch.allclose(gx, gxb, atol=2e-4), (gx - gxb).abs().max()
        for n in gb:
            scale = gb[n].abs().max().item() + 1e-6
            assert (g[n] - gb[n]).abs().max().item() / scale < 1e-4, n


def _accumulate(rank, world, use_scheduler):
    """Two micro-batches accumulated into one gradient: with the scheduler (full mode, trickled
    all-reduce) the first runs inside ``no_sync()``; without it gradients add up in ``param.grad``
    and are reduced once at the end."""
    from fluidmoe_b200.distributed import init_parallel
    from fluidmoe_b200.models.transformer import TransformerLayer
    from fluidmoe_b200.ops.rope import make_rope_freqs
    from fluidmoe_b200.parallel.scheduler import get_backward_scheduler

    H, nh, nkv, F, E, k, s_loc, b = 64, 4, 2, 96, 4, 2, 16, 2
    pc = init_parallel()
    torch.manual_seed(1)
    layer = TransformerLayer(H, nh, nkv, F, E, k, pc.cp_group, pc.ep_group, comm_mode="p2p", moe_combine_chunks=2,
                             moe_dispatch_chunks=2, attn_proj_chunks=2, attn_qkv_chunks=2, dtype=torch.float32,
                             device="cpu", router_dtype=torch.float32, norm_type="rmsnorm", init_std=0.2)
    rot = make_rope_freqs(world * s_loc, H // nh)
    sched = get_backward_scheduler()
    sched.configure_allreduce(use_scheduler, pc.dp_cp_group, pc.expert_dp_group,
                              gap_budgets={r: 1.0 for r in ("moe_combine", "moe_dispatch", "attn_proj", "attn_qkv")},
                              shared_ar_bw=1e6, expert_ar_bw=1e6)
    if use_scheduler:
        sched.enable(torch.device("cpu"))
        sched.eager_ar, sched.eager_ar_min_bytes = True, 0     # reduce as early as the policy allows
        expert = [layer.moe_w2, layer.moe_w1]
        sched.setup_ar_buffer([p for p in layer.parameters() if all(p is not e for e in expert)], True)
        sched.setup_expert_ar_buffer(expert, True)
    else:
        sched.disable()
    torch.manual_seed(20 + rank)
    batches = [(torch.randn(s_loc, b, H), torch.randn(s_loc, b, H)) for _ in range(2)]
    for i, (x, g) in enumerate(batches):
        x = x.requires_grad_(True)
        if use_scheduler and i == 0:
            with sched.no_sync():
                layer(x, rot).backward(g)
        else:
            layer(x, rot).backward(g)
    if use_scheduler:
        sched.finish_batch()
        grads = {n: p.main_grad.clone() for n, p in layer.named_parameters()}
    else:
        sched.sync_allreduce_params(list(layer.parameters()))
        grads = {n: p.grad.clone() for n, p in layer.named_parameters()}
    sched.clear_iteration()
    return grads


def test_gradient_accumulation_with_no_sync_world2():
    base = run_distributed(_accumulate, 2, False)
    got = run_distributed(_accumulate, 2, True)
    for r in range(2):
        for n in base[r]:
            scale = base[r][n].abs().max().item() + 1e-9
            assert (got[r][n] - base[r][n]).abs().max().item() / scale < 1e-4, (n, r)
