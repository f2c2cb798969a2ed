"""Public names outside the layer itself: the functional expert-parallel forward with uniform and
variable splits, the padding helper, the Megatron spec adapter (against stand-in ``megatron``
modules) and every import path of the compatibility package ``fluid``."""
import sys
import types

import pytest
import torch

from tests.dist_utils import run_distributed


# ------------------------------------------------------------------------------------------------
# moe_multicard_p2p_overlap_forward
# ------------------------------------------------------------------------------------------------
def _functional_forward(rank, world, variable):
    """Every rank routes T tokens to E experts; the functional entry point must return, for each
    permuted row, FC2(act(FC1(row)) * prob) of the expert that owns the row."""
    import torch.distributed as dist
    from fluidmoe_b200.distributed import init_parallel
    from fluidmoe_b200.models.moe import moe_multicard_p2p_overlap_forward
    from fluidmoe_b200.parallel.schedule import MultiCardOverlapContext

    pc = init_parallel()
    H, F, E = 32, 48, 4
    nle = E // world
    torch.manual_seed(5)
    w1_full = torch.randn(E, H, F) * 0.2
    w2_full = torch.randn(E, F, H) * 0.2
    w1, w2 = w1_full[rank * nle:(rank + 1) * nle].contiguous(), w2_full[rank * nle:(rank + 1) * nle].contiguous()
    g = torch.Generator().manual_seed(100 + rank)
    if variable:
        counts = torch.randint(1, 9, (E,), generator=g)          # rows this rank sends to every global expert
    else:
        counts = torch.full((E,), 6)
    rows = int(counts.sum())
    tokens = torch.randn(rows, H, generator=g)
    probs = torch.rand(rows, generator=g)
    input_splits = [int(counts[p * nle:(p + 1) * nle].sum()) for p in range(world)]
    # exchange the per-expert counts: row r of `all_counts` is what rank r sends
    all_counts = [torch.zeros(E, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(all_counts, counts.to(torch.int64))
    recv_counts = torch.stack([c[rank * nle:(rank + 1) * nle] for c in all_counts])     # [P, nle]
    output_splits = [int(recv_counts[p].sum()) for p in range(world)]
    ctx = MultiCardOverlapContext(torch.device("cpu"), world, world)
    out = moe_multicard_p2p_overlap_forward(
        tokens, input_splits, output_splits, w1, w2, pc.ep_group, "gelu", ctx, 0, nle,
        num_global_tokens_per_local_expert=recv_counts if variable else None, probs=probs)
    # oracle: every row with the full weights, no communication
    expert_of_row = torch.repeat_interleave(torch.arange(E), counts)
    ref = torch.empty_like(tokens)
    for e in range(E):
        sel = expert_of_row == e
        ref[sel] = (torch.nn.functional.gelu(tokens[sel] @ w1_full[e]) * probs[sel].unsqueeze(1)) @ w2_full[e]
    return (out - ref).abs().max().item(), ref.abs().max().item()


@pytest.mark.parametrize("variable", [False, True])
def test_functional_overlap_forward_matches_dense_experts_world2(variable):
    for err, scale in run_distributed(_functional_forward, 2, variable):
        assert err / scale < 1e-5, (err, scale)


# ------------------------------------------------------------------------------------------------
# pad_moe_dispatch
# ------------------------------------------------------------------------------------------------
def test_pad_moe_dispatch_pads_and_truncates():
    from fluidmoe_b200.models.moe import pad_moe_dispatch
    counts = torch.tensor([2, 0, 5, 3])
    tokens = torch.arange(10, dtype=torch.float32).unsqueeze(1).repeat(1, 3) + 1.0     # row i holds i + 1
    probs = torch.arange(10, dtype=torch.float32) + 0.5
    out, p, valid = pad_moe_dispatch(tokens, counts, 3, probs)
    assert out.shape == (12, 3) and p.shape == (12,) and valid.shape == (12,)
    expect_rows = [1, 2, 0, 0, 0, 0, 3, 4, 5, 8, 9, 10]        # expert 2 truncated to 3 of its 5 rows
    assert out[:, 0].tolist() == [float(v) for v in expect_rows]
    assert valid.tolist() == [v != 0 for v in expect_rows]
    assert torch.equal(p, torch.where(valid, torch.tensor(expect_rows, dtype=torch.float32) - 0.5, torch.zeros(12)))
    out2, valid2 = pad_moe_dispatch(tokens, counts, 3)
    assert torch.equal(out2, out) and torch.equal(valid2, valid)


# ------------------------------------------------------------------------------------------------
# Megatron adapter
# ------------------------------------------------------------------------------------------------
class _Cfg:
    hidden_size, num_attention_heads, num_query_groups = 64, 4, 2
    ffn_hidden_size, moe_ffn_hidden_size = 256, 96
    num_moe_experts, moe_router_topk, num_layers = 4, 2, 8
    gated_linear_unit, normalization, layernorm_epsilon = True, "RMSNorm", 1e-6
    moe_expert_capacity_factor, init_method_std = 1.25, 0.01
    params_dtype, moe_router_dtype = torch.float32, "fp32"
    moe_aux_loss_coeff, moe_z_loss_coeff = 1e-2, None

    @staticmethod
    def activation_func(x):
        return torch.nn.functional.silu(x)


_Cfg.activation_func.__name__ = "silu"


def test_layer_kwargs_from_config(monkeypatch):
    from fluidmoe_b200.models.megatron_spec import layer_kwargs_from_config
    from fluidmoe_b200.models.transformer import TransformerLayer
    monkeypatch.setenv("FLUIDMOE_MOE_COMBINE_CHUNKS", "4")
    monkeypatch.setenv("FLUIDMOE_ATTN_QKV_CHUNKS", "2")
    kw = layer_kwargs_from_config(_Cfg(), layer_number=3)
    assert kw["hidden_size"] == 64 and kw["num_heads"] == 4 and kw["num_kv_heads"] == 2
    assert kw["ffn_hidden_size"] == 96 and kw["num_experts"] == 4 and kw["top_k"] == 2 and kw["layer_id"] == 2
    assert kw["moe_combine_chunks"] == 4 and kw["attn_qkv_chunks"] == 2 and kw["moe_dispatch_chunks"] == 1
    assert kw["activation_func"] == "swiglu" and kw["norm_type"] == "rmsnorm" and kw["norm_eps"] == 1e-6
    assert kw["capacity_factor"] == 1.25 and kw["router_dtype"] == torch.float32
    assert abs(kw["output_init_std"] - 0.01 / 4.0) < 1e-12 and kw["aux_loss_coeff"] == 1e-2 and kw["z_loss_coeff"] == 0.0
    layer = TransformerLayer(device="cpu", **kw)          # the dictionary is a complete constructor call
    y = layer(torch.randn(8, 1, 64))
    assert y.shape == (8, 1, 64) and layer.moe_w1.shape == (4, 64, 192)


def test_megatron_layer_spec_with_stand_in_megatron(monkeypatch):
    """With stand-ins for ``megatron.core`` the spec builds, the module wraps a TransformerLayer on
    the groups Megatron hands out and returns ``(output, context)`` like a Megatron layer."""
    from fluidmoe_b200.models import megatron_spec

    def module(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        monkeypatch.setitem(sys.modules, name, m)
        return m

    class MegatronModule(torch.nn.Module):
        def __init__(self, config=None):
            super().__init__()
            self.config = config

    class ModuleSpec:
        def __init__(self, module=None, submodules=None):
            self.module, self.submodules = module, submodules

    ps = module("megatron.core.parallel_state", get_context_parallel_group=lambda: None,
                get_expert_model_parallel_group=lambda: None)
    module("megatron")
    module("megatron.core", parallel_state=ps)
    module("megatron.core.transformer")
    module("megatron.core.transformer.module", MegatronModule=MegatronModule)
    module("megatron.core.transformer.spec_utils", ModuleSpec=ModuleSpec)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    real_device = torch.device
    monkeypatch.setattr(megatron_spec.torch, "device", lambda *a, **k: real_device("cpu"))
    spec = megatron_spec.get_fluid_custom_layers()
    assert isinstance(spec, ModuleSpec)
    mod = spec.module(_Cfg(), layer_number=2)
    out, context = mod(torch.randn(8, 1, 64), rotary_pos_emb=(None,))
    assert out.shape == (8, 1, 64) and context is None
    assert set(mod.sharded_state_dict(prefix="decoder.layers.1.")) >= {"decoder.layers.1.layer.qkv_weight",
                                                                        "decoder.layers.1.layer.moe_w1"}


def test_megatron_layer_spec_without_megatron_raises():
    from fluidmoe_b200.models import megatron_spec
    if "megatron" in sys.modules:
        pytest.skip("megatron importable")
    with pytest.raises(ImportError, match="megatron-core"):
        megatron_spec.get_fluid_gpt_layer_spec()


# ------------------------------------------------------------------------------------------------
# compatibility import paths
# ------------------------------------------------------------------------------------------------
def test_reference_import_paths_resolve():
    import importlib
    fluid = importlib.import_module("fluid")
    for name in fluid.__all__:
        assert hasattr(fluid, name), name
    # the names the reference exports (fluid/__init__.py:90-131)
    exported = """_all_to_all _all_to_all_sp2hp_forward _all_to_all_hp2sp_forward MultiCardOverlapContext
        BackwardScheduler get_p2p_backend get_backward_scheduler router_forward dispatch_fc1_p2p_forward
        fc2_combine_p2p_forward combine_fc2_backward fc1_dispatch_backward register_moe_dw_tasks router_backward
        register_router_dw_task qkv_projection_p2p_forward scaled_dot_product_attention_forward
        output_projection_p2p_forward outproj_sp2hp_backward hp2sp_qkv_backward output_projection_register_dw
        TransformerLayerFunction TransformerLayer TransformerModel FluidDDP FluidOptimizerWrapper
        setup_model_and_optimizer""".split()
    missing = [n for n in exported if n not in fluid.__all__ or not callable(getattr(fluid, n, None))]
    assert not missing, missing
    ns = {}
    exec("from fluid import *", ns)          # star import honours the export list
    assert "_all_to_all" in ns and "TransformerLayer" in ns
    from fluid import (FluidDDP, FluidOptimizerWrapper, MoEBaseline, MultiCardOverlapContext,  # noqa: F401
                       TransformerLayer, TransformerLayerFunction, TransformerModel, get_backward_scheduler,
                       get_fluid_custom_layers, get_p2p_backend, moe_multicard_p2p_overlap_forward,
                       setup_model_and_optimizer)
    from fluid.attention import CPPlan, qkv_projection_p2p_forward, output_projection_p2p_forward  # noqa: F401
    from fluid.attention.backward import hp2sp_qkv_backward, outproj_sp2hp_backward  # noqa: F401
    from fluid.attention.forward import scaled_dot_product_attention_forward  # noqa: F401
    from fluid.core import compute_round_robin_schedule  # noqa: F401
    from fluid.core.comm import _all_to_all, _all_to_all_hp2sp_forward, _all_to_all_sp2hp_forward  # noqa: F401
    from fluid.core.nvtx import nvtx_range, nvtx_range_pop, nvtx_range_push  # noqa: F401
    from fluid.core.overhead_profiler import get_overhead_profiler  # noqa: F401
    from fluid.core.p2p_backend import NCCLBackend, NVSHMEMBackend, P2PBackend, reset_p2p_backend  # noqa: F401
    from fluid.core.python_profile import get_profile_stats, profile_section, reset_profile_stats  # noqa: F401
    from fluid.core.scheduler import BackwardScheduler  # noqa: F401
    from fluid.core.stream import get_stream_manager  # noqa: F401
    from fluid.core.te_ops import te_dgelu, te_gelu, te_layernorm_bwd, te_layernorm_fwd_with_stats, te_silu  # noqa: F401
    from fluid.distributed import init_parallel  # noqa: F401
    from fluid.layer.fluid_spec import get_fluid_gpt_layer_spec  # noqa: F401
    from fluid.layer.transformer import TransformerLayer as TL2  # noqa: F401
    from fluid.moe import (EPPlan, build_moe_chunk_config, combine_fc2_backward, dispatch_fc1_p2p_forward,  # noqa: F401
                           fc1_dispatch_backward, fc2_combine_p2p_forward, grouped_fc1_act, grouped_fc1_dx,
                           grouped_fc2, grouped_fc2_dx, pad_moe_dispatch, register_moe_dw_tasks,
                           register_router_dw_task, router_backward, router_forward)
    from fluid.setup import FluidDDP as DDP2  # noqa: F401
    assert TL2 is TransformerLayer and DDP2 is FluidDDP
    assert compute_round_robin_schedule(8)[0] == [(0, 7), (1, 6), (2, 5), (3, 4)]
    assert fluid.__version__ == "1.0.0"


def test_embedding_backward_adds_touched_rows_into_the_gradient_buffer():
    """``models.gpt._Embedding``: with an fp32 ``main_grad`` on the weight the touched rows are added
    there and no dense gradient is produced; without one the dense gradient equals ``F.embedding``'s."""
    import torch
    import torch.nn.functional as F
    from fluidmoe_b200.models.gpt import _Embedding

    torch.manual_seed(0)
    V, H = 50, 16
    ids = torch.randint(0, V, (12, 3))
    ids[0, 0] = ids[1, 1] = 7                      # a repeated row
    gy = torch.randn(12, 3, H)
    w_ref = torch.randn(V, H, requires_grad=True)
    F.embedding(ids, w_ref).backward(gy)

    w = w_ref.detach().clone().requires_grad_(True)
    y = _Embedding.apply(ids, w)
    assert torch.equal(y, F.embedding(ids, w_ref))
    y.backward(gy)
    assert torch.allclose(w.grad, w_ref.grad, atol=1e-6)

    w2 = w_ref.detach().clone().requires_grad_(True)
    w2.main_grad = torch.ones(V, H)                # accumulates on top of what is there
    _Embedding.apply(ids, w2).backward(gy)
    assert w2.grad is None
    assert torch.allclose(w2.main_grad, 1.0 + w_ref.grad, atol=1e-6)


def test_flat_gradient_buffer_cursors():
    """write / committed / read cursors of the flat gradient buffer: `has_remainder` counts what is
    written but not committed too, `has_pending` only what the all-reduce may take."""
    from fluidmoe_b200.parallel.scheduler import FlatGradBuffer
    a, b = torch.nn.Parameter(torch.zeros(4)), torch.nn.Parameter(torch.zeros(6))
    buf = FlatGradBuffer()
    buf.setup([a, b])
    assert not buf.has_remainder() and not buf.has_pending()
    buf.write_grad(b, torch.ones(6))                 # out of layout order: the prefix is not complete yet
    assert not buf.has_remainder()
    buf.write_grad(a, torch.ones(4))
    assert buf.has_remainder() and not buf.has_pending() and buf.pending_bytes() == 0
    buf.commit()
    assert buf.has_pending() and buf.pending_bytes() == 10 * 4
    seen = []
    buf.submit_block(lambda t, scale: seen.append(t.numel()))
    assert seen == [10] and not buf.has_pending() and not buf.has_remainder()


def test_optimizer_wrapper_passes_public_attributes_through():
    """Reads and writes of public attributes reach the wrapped optimizer (fluid/setup.py:403-410);
    `step` resets the scheduler's iteration state; the DDP wrapper accepts Megatron's
    `finish_grad_sync(force_all_reduce=...)` spelling."""
    import inspect
    import fluidmoe_b200 as fm

    class _Sched:
        cleared = 0

        def clear_iteration(self):
            self.cleared += 1

    lin = torch.nn.Linear(3, 2)
    inner = torch.optim.SGD(lin.parameters(), lr=0.1)
    sched = _Sched()
    opt = fm.FluidOptimizerWrapper(inner, sched)
    assert opt.optimizer is inner and opt.scheduler is sched
    assert opt.param_groups is inner.param_groups
    opt.my_flag = 7
    assert inner.my_flag == 7 and "my_flag" not in vars(opt)
    lin(torch.ones(1, 3)).sum().backward()
    opt.step()
    assert sched.cleared == 1
    opt.zero_grad()
    assert all(p.grad is None or float(p.grad.abs().sum()) == 0.0 for p in lin.parameters())
    assert opt.state_dict().keys() == inner.state_dict().keys()
    assert "force_all_reduce" in inspect.signature(fm.FluidDDP.finish_grad_sync).parameters


def test_compat_helpers_of_comm_backend_and_stream_modules(monkeypatch):
    """Small names of the reference's core modules: the all-to-all-v split checker, the NVLink probe
    and the stream manager's one-sided transport hooks."""
    import fluid.core.comm as c
    import fluid.core.p2p_backend as p
    import fluid.core.stream as st
    from fluidmoe_b200.parallel.comm import SplitMismatchError
    c._debug_check_alltoallv_splits(4, 4, [1, 2], [3, 3], None, "off")        # disabled: nothing is checked
    monkeypatch.setenv("FLUID_DEBUG_A2A_SPLITS", "1")
    c._debug_check_alltoallv_splits(4, 4, [4], [4], None, "ok")               # one rank, consistent
    c._debug_check_alltoallv_splits(4, 4, None, [4], None, "no lists")
    with pytest.raises(SplitMismatchError, match="2 input"):
        c._debug_check_alltoallv_splits(4, 4, [2, 2], [4], None, "len")
    with pytest.raises(SplitMismatchError, match="add up to 3"):
        c._debug_check_alltoallv_splits(4, 4, [3], [4], None, "sum")
    with pytest.raises(SplitMismatchError, match="output splits add up to 5"):
        c._debug_check_alltoallv_splits(4, 4, [4], [5], None, "sum")
    assert p._has_nvlink() in (True, False)
    mgr = st.StreamManager()
    assert mgr.nvshmem_initialized is False
    with pytest.raises(RuntimeError, match="CUDA device"):
        mgr.init_nvshmem()


def test_moe_backward_helpers_under_reference_names(monkeypatch):
    """`recompute_fc1_gemm` (fluid/moe/backward.py:616-646) against a per-expert matmul, the dW
    ablation probes, and the grouped-GEMM aliases of the forward / backward submodules."""
    import fluid.moe.backward as mb
    import fluid.moe.forward as mf
    import fluid.layer.fluid_spec as spec
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler
    torch.manual_seed(0)
    counts = [3, 0, 5]
    tokens = torch.randn(8, 16)
    w1 = torch.randn(3, 16, 24)
    pre = mb.recompute_fc1_gemm(tokens, counts, w1)
    ref = torch.cat([tokens[0:3] @ w1[0], tokens[3:8] @ w1[2]])
    assert torch.allclose(pre, ref, atol=1e-5)
    assert mb.recompute_fc1_gemm(tokens[:0], [0, 0, 0], w1).shape == (0, 24)
    assert mb.skip_all_dw() is False and mb.skip_dispatch_dw() is False
    s = BackwardScheduler()                      # the process-wide scheduler; the flags start from the environment
    monkeypatch.setattr(s, "skip_all_dw", True)
    monkeypatch.setattr(s, "skip_dispatch_dw", True)
    assert mb.skip_all_dw() is True and mb.skip_dispatch_dw() is True
    assert callable(mf.grouped_fc1_act) and callable(mf.grouped_fc2)
    assert callable(mb.grouped_fc1_dx) and callable(mb.grouped_fc2_dx)
    if "megatron" not in sys.modules:
        with pytest.raises(ImportError, match="megatron-core"):
            spec.FluidTransformerLayer


def test_one_sided_extension_names_resolve_and_guard_their_state():
    """`fluid.csrc` offers the entry points of the reference's extension
    (fluid/csrc/nvshmem_ops.cpp:268-289); before initialisation every call that needs the heap says so."""
    import fluid.csrc as c
    for name in """nvshmem_init nvshmem_init_with_uniqueid nvshmem_get_uniqueid nvshmem_uniqueid_size nvshmem_finalize
                   nvshmem_my_pe nvshmem_n_pes nvshmem_malloc_tensor nvshmem_free_tensor nvshmem_ptr
                   putmem_signal_on_stream signal_wait_until_on_stream quiet_on_stream SIGNAL_SET CMP_GE""".split():
        assert callable(getattr(c, name)), name
    assert len(c.nvshmem_get_uniqueid()) == c.nvshmem_uniqueid_size()
    assert c.nvshmem_is_initialized() is False
    for call in (c.nvshmem_my_pe, c.nvshmem_n_pes, lambda: c.nvshmem_malloc_tensor(8, torch.float32),
                 lambda: c.nvshmem_ptr(torch.zeros(4), 0), lambda: c.quiet_on_stream(0),
                 lambda: c.putmem_signal_on_stream(16, torch.zeros(4), 16, 16, 1, c.SIGNAL_SET(), 0, 0),
                 lambda: c.signal_wait_until_on_stream(16, c.CMP_GE(), 1, 0)):
        with pytest.raises(RuntimeError, match="not initialised"):
            call()
    with pytest.raises(ValueError, match="does not match"):
        c.nvshmem_init_with_uniqueid(3, 8, c.nvshmem_get_uniqueid())      # this process is rank 0 of 1
    with pytest.raises(ValueError, match="unique id"):
        c.nvshmem_init_with_uniqueid(0, 1, b"short")
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="CUDA device"):
            c.nvshmem_init()
    c.nvshmem_finalize()                                                   # harmless when nothing is mapped
