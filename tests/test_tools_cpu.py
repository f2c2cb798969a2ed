"""Presets, persistence of tuned defaults, chunk planning, schedule properties and the block
benchmark driver (single process, CPU)."""
import json
import os

import pytest
import torch


def test_model_presets_match_reference_shapes():
    from fluidmoe_b200.tools.model_configs import get_model_config, list_model_names
    m = get_model_config("mixtral_8x7b")
    assert (m["hidden_size"], m["num_heads"], m["num_kv_heads"], m["ffn_hidden"], m["num_experts"], m["top_k"]) == \
        (4096, 32, 8, 14336, 8, 2)
    assert {"dbrx", "phi_3_5_moe", "olmoe_1b_7b", "deepseek_v3_mha_proxy", "glm4_5_air_mha_proxy"} <= set(list_model_names())
    with pytest.raises(KeyError):
        get_model_config("nope")


def test_tuned_defaults_round_trip(tmp_path, monkeypatch):
    from fluidmoe_b200.tools import experiment_configs as ec
    monkeypatch.setenv("FLUIDMOE_TUNED_DEFAULTS", str(tmp_path / "t.json"))
    assert ec.get_block_benchmark_defaults()["moe_combine_chunks"] == 2
    ec.persist_block_benchmark_defaults({"moe_combine_chunks": 4, "gap_budgets": {"attn_qkv": 0.9}})
    cfg = ec.get_block_benchmark_defaults()
    assert cfg["moe_combine_chunks"] == 4 and cfg["gap_budgets"]["attn_qkv"] == 0.9
    assert cfg["gap_budgets"]["moe_combine"] == 0.5          # untouched keys keep their defaults
    assert json.load(open(tmp_path / "t.json"))["default"]["moe_combine_chunks"] == 4


def test_chunk_decomposition():
    from fluidmoe_b200.models.moe import build_region_chunk_config, decompose_chunks
    assert decompose_chunks(4, 1, 1024) == (1, 4)          # one local expert: capacity dimension only
    assert decompose_chunks(4, 8, 768) == (4, 1)           # expert dimension first
    assert decompose_chunks(8, 2, 96) == (2, 4)
    assert decompose_chunks(4, 1, 1023) == (1, 3)          # falls back to a divisor of the capacity
    c = build_region_chunk_config(8, 8, 100)
    assert c.mode == "expert" and c.skip_index and c.num_chunks == 8


def test_round_robin_schedule_properties():
    from fluidmoe_b200.parallel.schedule import MultiCardOverlapContext, compute_round_robin_schedule
    s8 = compute_round_robin_schedule(8)
    assert len(s8) == 7 and s8[0] == [(0, 7), (1, 6), (2, 5), (3, 4)]
    for P in range(2, 10):
        sched = compute_round_robin_schedule(P)
        assert len(sched) == (P - 1 if P % 2 == 0 else P)
        seen = set()
        for rnd in sched:
            busy = [r for pair in rnd for r in pair]
            assert len(busy) == len(set(busy))
            seen |= set(rnd)
        assert len(seen) == P * (P - 1) // 2
    ctx = MultiCardOverlapContext(torch.device("cpu"), 5)
    assert ctx.num_rounds == 5 and sum(ctx.get_partner(0, r) == -1 for r in range(5)) == 1


def test_scheduler_queue_policy():
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler
    BackwardScheduler.reset()
    s = BackwardScheduler()
    s.enable(torch.device("cpu"))
    ran = []
    for i in range(5):
        s.register_dw_task(f"t{i}", 0, (lambda i=i: ran.append(i)), None, defer=(i != 3))
    assert s.execute_dw_tasks(max_defer_tasks=2) == 3       # two deferrable + the non-deferrable one
    assert ran == [0, 1, 3]
    s.finish_batch()
    assert ran == [0, 1, 3, 2, 4]                            # leftovers kept their order
    BackwardScheduler.reset()


def test_block_benchmark_driver_runs_on_cpu(capsys):
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler
    from fluidmoe_b200.tools import run_block_benchmark
    BackwardScheduler.reset()
    run_block_benchmark.main(["--model", "tiny_test", "--impl", "fluidmoe-fb", "--warmup", "1", "--iters", "1"])
    out = capsys.readouterr().out
    assert "RESULT impl=fluidmoe-fb" in out and "tokens_per_sec=" in out
    BackwardScheduler.reset()


def test_checkpoint_round_trip(tmp_path):
    from fluidmoe_b200.models.transformer import TransformerModel
    from fluidmoe_b200.utils.checkpoint import load_checkpoint, load_reference_state_dict, save_checkpoint
    kw = dict(dtype=torch.float32, device="cpu")
    a = TransformerModel(2, 64, 4, 2, 96, 4, 2, **kw)
    b = TransformerModel(2, 64, 4, 2, 96, 4, 2, **kw)
    keys = set(a.state_dict())
    assert {"layers.0.ln1_weight", "layers.0.ln1_bias", "layers.0.qkv_weight", "layers.0.proj_weight",
            "layers.0.router_weight", "layers.0.moe_w1", "layers.1.moe_w2"} <= keys
    assert a.state_dict()["layers.0.qkv_weight"].shape == (2 * (2 + 2) * 16, 64)
    assert a.state_dict()["layers.0.moe_w1"].shape == (4, 64, 96)
    save_checkpoint(a, str(tmp_path / "ck"), step=7)
    man = load_checkpoint(b, str(tmp_path / "ck"))
    assert man["step"] == 7
    x = torch.randn(8, 1, 64)
    assert torch.equal(a(x), b(x))
    sd = {k.replace("qkv_weight", "te_qkv_linear.weight"): v for k, v in a.state_dict().items()}
    sd["layers.0.te_attn._extra_state"] = torch.zeros(1)
    load_reference_state_dict(b, sd)


def _train_steps(model, opt, xs):
    for x in xs:
        for p in model.parameters():
            p.grad = None
        model(x).square().mean().backward()
        opt.step()


def test_checkpoint_resume_with_optimizer_matches_uninterrupted_run(tmp_path):
    """Two steps, save, load into a fresh model + optimizer, two more steps == four steps in one go;
    the loaded moments live on the parameter's device in the optimizer's state dtype."""
    from fluidmoe_b200.models.transformer import TransformerModel
    from fluidmoe_b200.ops.optim import FusedAdam
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler
    from fluidmoe_b200.utils.checkpoint import load_checkpoint, reshard_experts, save_checkpoint
    BackwardScheduler.reset()
    kw = dict(dtype=torch.float32, device="cpu")
    torch.manual_seed(3)
    xs = [torch.randn(8, 1, 64) for _ in range(4)]
    torch.manual_seed(4)
    a = TransformerModel(1, 64, 4, 2, 96, 4, 2, **kw)
    oa = FusedAdam(a.parameters(), lr=1e-2)
    _train_steps(a, oa, xs[:2])
    save_checkpoint(a, str(tmp_path / "ck"), optimizer=oa, step=2)
    _train_steps(a, oa, xs[2:])
    torch.manual_seed(5)
    b = TransformerModel(1, 64, 4, 2, 96, 4, 2, **kw)
    ob = FusedAdam(b.parameters(), lr=1e-2)
    load_checkpoint(b, str(tmp_path / "ck"), optimizer=ob)
    assert ob.step_count == 2
    for p in ob.params:
        st = ob.state[id(p)]
        assert st["m"].device == p.device and st["m"].dtype == ob.state_dtype and st["m"].shape == p.shape
    _train_steps(b, ob, xs[2:])
    for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.allclose(pa, pb, atol=1e-6), n
    # a state tensor of the wrong shape is refused
    bad = oa.state_dict()
    bad["state"][0]["m"] = torch.zeros(3)
    with pytest.raises(ValueError, match="shape"):
        FusedAdam(b.parameters()).load_state_dict(bad)
    # resharding keeps the optimizer state and splits expert moments along the expert dimension
    reshard_experts(str(tmp_path / "ck"), str(tmp_path / "ck2"), 2)
    s0 = torch.load(str(tmp_path / "ck2" / "shard_ep000.pt"))
    s1 = torch.load(str(tmp_path / "ck2" / "shard_ep001.pt"))
    names = s0["optimizer_param_names"]
    i = names.index("layers.0.moe_w1")
    full = torch.load(str(tmp_path / "ck" / "shard_ep000.pt"))["optimizer"]["state"][i]["m"]
    assert torch.equal(torch.cat([s0["optimizer"]["state"][i]["m"], s1["optimizer"]["state"][i]["m"]]), full)
    j = names.index("layers.0.qkv_weight")
    assert torch.equal(s0["optimizer"]["state"][j]["v"], s1["optimizer"]["state"][j]["v"])
    BackwardScheduler.reset()


def test_comm_timer_counts_and_restores():
    """The collective timers wrap the torch.distributed entry points only inside the context."""
    import torch.distributed as dist
    from fluidmoe_b200.tools import comm_ratio_table as crt
    orig = dist.all_reduce
    seen = []

    def fake_all_reduce(t, *a, **k):
        seen.append(t.numel())
    dist.all_reduce = fake_all_reduce
    try:
        iter_ms, table = crt.measure(lambda: dist.all_reduce(torch.zeros(4)), 3, torch.device("cpu"))
        assert dist.all_reduce is fake_all_reduce          # restored
    finally:
        dist.all_reduce = orig
    assert seen == [4, 4, 4]
    assert table["all_reduce"][0] == 1.0 and table["all_reduce"][1] >= 0.0
    text = crt.format_table(max(iter_ms, 1e-6), table)
    assert "all_reduce" in text and "iteration" in text


def test_comm_ratio_table_runs_on_cpu(capsys):
    from fluidmoe_b200.tools import comm_ratio_table as crt
    crt.main(["--model", "tiny_test", "--iters", "1", "--warmup", "1"])
    assert "iteration" in capsys.readouterr().out


def test_profile_capture_writes_table(tmp_path, capsys):
    from fluidmoe_b200.tools import profile_capture
    out = tmp_path / "table.txt"
    profile_capture.main(["--model", "tiny_test", "--impl", "fluidmoe-fb", "--warmup", "1", "--iters", "1",
                          "--table", str(out)])
    assert "captured 1 iteration" in capsys.readouterr().out
    assert out.read_text().strip()


def test_external_baselines_report_missing_packages():
    from fluidmoe_b200.tools import external_baselines as eb
    from fluidmoe_b200.tools.model_configs import get_model_config
    avail = eb.available()
    assert set(avail) == {"megatron", "deepspeed"}
    cfg = get_model_config("tiny_test")
    if not avail["megatron"]:
        with pytest.raises(eb.BaselineUnavailable, match="package"):
            eb.build_megatron_baseline(cfg, device="cpu")
    if not avail["deepspeed"]:
        with pytest.raises(eb.BaselineUnavailable, match="package"):
            eb.build_deepspeed_ulysses_baseline(cfg, device="cpu")


def test_external_baselines_build_with_stub_packages(monkeypatch):
    """With stand-ins for megatron-core / transformer_engine / deepspeed on the import path both
    builders run to the end for every preset: the preset keys they read exist and the arguments
    they pass are the ones the packages' constructors take."""
    import sys
    import types
    from fluidmoe_b200.tools import external_baselines as eb
    from fluidmoe_b200.tools.model_configs import get_model_config, list_model_names

    seen = {}

    def module(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        monkeypatch.setitem(sys.modules, name, m)
        return m

    class TransformerConfig:
        def __init__(self, **kw):
            seen["tc"] = kw

    class TransformerBlock(torch.nn.Module):
        def __init__(self, config, spec, post_layer_norm=True):
            super().__init__()
            seen["block"] = (config, spec, post_layer_norm)

    module("megatron")
    module("megatron.core")
    module("transformer_engine")
    module("megatron.core.models")
    module("megatron.core.models.gpt")
    module("megatron.core.models.gpt.gpt_layer_specs",
           get_gpt_layer_with_transformer_engine_spec=lambda **kw: ("spec", kw))
    module("megatron.core.transformer")
    module("megatron.core.transformer.transformer_block", TransformerBlock=TransformerBlock)
    module("megatron.core.transformer.transformer_config", TransformerConfig=TransformerConfig)

    class MoE(torch.nn.Module):
        def __init__(self, hidden, expert, num_experts, ep_size, k, capacity_factor, drop_tokens):
            super().__init__()
            seen["moe"] = dict(hidden=hidden, num_experts=num_experts, ep_size=ep_size, k=k,
                               capacity_factor=capacity_factor, ffn=expert[0].out_features)

    class DistributedAttention(torch.nn.Module):
        def __init__(self, local, group, scatter_idx, gather_idx):
            super().__init__()
            self.local = local

    module("deepspeed")
    module("deepspeed.moe")
    module("deepspeed.moe.layer", MoE=MoE)
    module("deepspeed.sequence")
    module("deepspeed.sequence.layer", DistributedAttention=DistributedAttention)

    assert eb.available() == {"megatron": True, "deepspeed": True}
    for name in list_model_names():
        cfg = get_model_config(name)
        eb.build_megatron_baseline(cfg, device="cpu")
        tc = seen["tc"]
        assert tc["ffn_hidden_size"] == cfg["ffn_hidden"] and tc["num_query_groups"] == cfg["num_kv_heads"]
        assert tc["normalization"] == ("RMSNorm" if cfg.get("norm_type") == "rmsnorm" else "LayerNorm")
        assert tc["gated_linear_unit"] == (cfg.get("activation") == "swiglu")
        assert tc["moe_token_dispatcher_type"] == "alltoall" and tc["cp_comm_type"] == "a2a"
    small = get_model_config("tiny_test")
    model = eb.build_deepspeed_ulysses_baseline(small, ep_size=1, dtype=torch.float32, device="cpu")
    assert len(model) == small["num_layers"]
    assert seen["moe"] == dict(hidden=small["hidden_size"], num_experts=small["num_experts"], ep_size=1,
                               k=small["top_k"], capacity_factor=1.0, ffn=small["ffn_hidden"])


def test_block_benchmark_runs_several_presets_and_halves(capsys, monkeypatch):
    """Several presets in one run: a MoE-only layer with a Zipf router prior and dropless routing,
    an attention-only block with RoPE, and the reference-expressible variant of a SwiGLU preset."""
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler
    from fluidmoe_b200.tools import model_configs, run_block_benchmark
    tiny = dict(hidden_size=128, num_heads=4, num_kv_heads=2, ffn_hidden=96, num_experts=8, top_k=2, num_layers=1,
                seq_len=64, seq_per_rank=64, batch_size=1, activation="swiglu", norm_type="rmsnorm")
    monkeypatch.setitem(model_configs.MODEL_CONFIGS, "t_moe", dict(tiny, capacity_factor=0.0, num_shared_experts=1,
                                                                   has_attention=False, zipf_s=1.1))
    monkeypatch.setitem(model_configs.MODEL_CONFIGS, "t_attn", dict(tiny, capacity_factor=1.0, has_moe=False, rope=True))
    BackwardScheduler.reset()
    run_block_benchmark.main(["--model", "t_moe,t_attn", "--impl", "fluidmoe-full", "--warmup", "1", "--iters", "1"])
    out = capsys.readouterr().out
    assert out.count("RESULT impl=fluidmoe-full") == 2 and "model=t_moe" in out and "model=t_attn" in out
    run_block_benchmark.main(["--model", "t_moe", "--impl", "fluidmoe-fb", "--matched", "--warmup", "1", "--iters", "1"])
    assert "RESULT impl=fluidmoe-fb-matched model=t_moe" in capsys.readouterr().out
    ref = model_configs.reference_variant(model_configs.get_model_config("t_moe"))
    assert ref["activation"] == "gelu" and ref["ffn_hidden"] == 144 and ref["capacity_factor"] == 1.0
    assert ref["num_shared_experts"] == 0 and ref["has_attention"] and ref["norm_type"] == "layernorm"
    BackwardScheduler.reset()


def test_tuner_searches_chunks_and_persists(tmp_path, monkeypatch, capsys):
    """The tuner's chunk search and gap profiling on one CPU process; results go to the JSON file."""
    import json
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler
    from fluidmoe_b200.tools import experiment_configs, tune
    monkeypatch.setenv("FLUIDMOE_TUNED_DEFAULTS", str(tmp_path / "tuned.json"))
    monkeypatch.setitem(experiment_configs.TUNE_DEFAULTS, "max_chunks", 2)
    monkeypatch.setitem(experiment_configs.TUNE_DEFAULTS, "iters", 1)
    monkeypatch.setitem(experiment_configs.TUNE_DEFAULTS, "warmup", 1)
    monkeypatch.setitem(experiment_configs.TUNE_DEFAULTS, "ar_sizes_mb", (1,))
    BackwardScheduler.reset()
    tune.main(["--model", "tiny_test", "--comm", "p2p", "--node-name", "testbox"])
    out = capsys.readouterr().out
    assert "[tune] all regions 1 chunk" in out and "[tune] wrote" in out
    saved = json.loads((tmp_path / "tuned.json").read_text())["testbox"]
    assert {"moe_combine_chunks", "moe_dispatch_chunks", "attn_proj_chunks", "attn_qkv_chunks",
            "shared_ar_bw", "gap_budgets"} <= set(saved)
    merged = experiment_configs.get_block_benchmark_defaults("testbox")
    assert merged["moe_combine_chunks"] == saved["moe_combine_chunks"]
    BackwardScheduler.reset()


def test_tuner_fused_knob_search_with_a_stub_timer(monkeypatch, capsys):
    """The knob search of the device-initiated transport: every trial reaches the timer with the
    knob names the search uses, and a knob is kept only when it saves at least ``min_saving_ms``."""
    import inspect
    from fluidmoe_b200.tools import tune
    # the real timer takes the knobs under the names the search passes
    assert list(inspect.signature(tune._time_fused).parameters)[5:] == ["eager_ar_min_bytes", "grad_reduce", "dw_side_ctas"]
    seen = []

    def fake_time(cfg, bench, pc, device, td, eager_ar_min_bytes, grad_reduce, dw_side_ctas):
        seen.append((eager_ar_min_bytes, grad_reduce, dw_side_ctas))
        return 10.0 - (1.0 if grad_reduce == "symm" else 0.0) - (0.01 if dw_side_ctas else 0.0)

    monkeypatch.setattr(tune, "_time_fused", fake_time)
    best = tune.tune_fused({}, {}, None, None, dict(min_saving_ms=0.05, side_ctas=(48,)))
    assert best == {"fused_eager_ar_min_bytes": 32 << 20, "fused_grad_reduce": "symm", "fused_dw_side_ctas": 0}
    assert len(seen) == 5 and seen[0] == (32 << 20, "nccl", 0)


def test_timeline_idle_gaps_and_collective_overlap():
    """The step profile's arithmetic: gaps that no stream fills, and how long a collective ran beside
    a kernel, counting a collective once although the profiler lists it as kernel and annotation."""
    from fluidmoe_b200.utils.timeline import idle_gaps, merge_intervals, overlap
    recs = [(0.0, 10.0, "a"), (12.0, 20.0, "b"), (15.0, 30.0, "side"), (30.0, 31.0, "c"), (40.0, 41.0, "d")]
    span, idle, gaps = idle_gaps(recs)
    assert span == 41.0 and idle == 2.0 + 9.0
    assert gaps == [(2.0, "a", "b"), (9.0, "c", "d")]          # b -> side -> c leaves no gap
    assert idle_gaps([]) == (0.0, 0.0, [])
    coll = merge_intervals([(5.0, 9.0), (5.0, 9.0), (8.0, 14.0), (20.0, 20.0), (25.0, 26.0)])
    assert coll == [(5.0, 14.0), (25.0, 26.0)]
    assert overlap(0.0, 10.0, coll) == 5.0 and overlap(12.0, 30.0, coll) == 3.0 and overlap(30.0, 40.0, coll) == 0.0


def test_driver_flags_shared_with_the_reference(capsys):
    """`--list-models`, the three parallel sizes and the chunk counts on the drivers
    (tests/run_block_benchmark.py:188-196 and the tools beside it)."""
    import argparse
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler
    from fluidmoe_b200.tools import common, overlap_ratio_analyzer, run_block_benchmark, tune
    for tool in (run_block_benchmark, overlap_ratio_analyzer, tune):
        tool.main(["--list-models"])
        out = capsys.readouterr().out
        assert "mixtral_8x7b" in out and "tiny_test" in out and "RESULT" not in out
    # sizes: any subset fixes the rest; contradictions are refused
    assert common.resolve_parallel_sizes(8) == (1, 8)
    assert common.resolve_parallel_sizes(8, dp_size=2) == (2, 4)
    assert common.resolve_parallel_sizes(8, cp_size=4, ep_size=4) == (2, 4)
    assert common.resolve_parallel_sizes(1, dp_size=1, cp_size=1, ep_size=1) == (1, 1)
    for bad in (dict(cp_size=4, ep_size=2), dict(dp_size=3), dict(dp_size=4, cp_size=4), dict(cp_size=3)):
        with pytest.raises(ValueError):
            common.resolve_parallel_sizes(8, **bad)
    # chunk counts from the command line replace the tuned defaults, the others stay
    ap = argparse.ArgumentParser()
    common.add_parallel_args(ap, chunks=True)
    args = ap.parse_args(["--moe-combine-chunks", "4", "--attn-qkv-chunks", "1"])
    bench = common.apply_chunk_args(args, dict(moe_combine_chunks=2, moe_dispatch_chunks=2, attn_proj_chunks=8, attn_qkv_chunks=4))
    assert bench == dict(moe_combine_chunks=4, moe_dispatch_chunks=2, attn_proj_chunks=8, attn_qkv_chunks=1)
    # and the block benchmark takes them (one process: every size is 1)
    BackwardScheduler.reset()
    run_block_benchmark.main(["--model", "tiny_test", "--impl", "fluidmoe-full", "--warmup", "1", "--iters", "1",
                              "--dp-size", "1", "--cp-size", "1", "--ep-size", "1", "--moe-dispatch-chunks", "1"])
    assert "RESULT impl=fluidmoe-full" in capsys.readouterr().out
    BackwardScheduler.reset()


def test_experiment_config_getters_return_copies():
    from fluidmoe_b200.tools import experiment_configs as ec
    td = ec.get_tune_defaults()
    td["max_chunks"] = -1
    assert ec.get_tune_defaults()["max_chunks"] == ec.TUNE_DEFAULTS["max_chunks"] != -1
    ds = ec.get_deepspeed_ulysses_defaults()
    assert ds["zero_stage"] == 0 and ds is not ec.DEEPSPEED_ULYSSES_DEFAULTS


def _parallel_sizes_worker(rank, world, flags):
    import argparse
    from fluidmoe_b200.parallel.scheduler import get_backward_scheduler
    from fluidmoe_b200.tools import common
    from fluidmoe_b200.tools.experiment_configs import get_block_benchmark_defaults
    ap = argparse.ArgumentParser()
    common.add_parallel_args(ap, chunks=True)
    args = ap.parse_args(flags)
    device, cfg, pc = common.setup("tiny_test", {"num_layers": 1}, "p2p", args=args)
    bench = common.apply_chunk_args(args, get_block_benchmark_defaults())
    model = common.build_model(cfg, bench, pc, device, "p2p", dtype=torch.float32)
    x = common.make_input(cfg, pc, device, dtype=torch.float32)
    sched = get_backward_scheduler()
    sched.enable(device)
    sched.configure_allreduce(True, pc.dp_cp_group, pc.expert_dp_group)
    model.setup_ar_buffer()
    common.run_iters(model, x, 1, pc)
    gnorm = sum(float(p.main_grad.float().pow(2).sum()) for p in model.parameters() if hasattr(p, "main_grad"))
    return dict(dp=pc.dp_size, cp=pc.cp_size, ep=pc.ep_size, rows=int(x.shape[0]), gnorm=gnorm)


@pytest.mark.parametrize("flags,dp,cp", [(["--dp-size", "2"], 2, 1), (["--cp-size", "2", "--ep-size", "2"], 1, 2),
                                         ([], 1, 2)])
def test_driver_parallel_sizes_on_two_ranks(flags, dp, cp):
    """Two gloo ranks as two data-parallel replicas, or as one sequence- and expert-parallel group:
    the groups are built as asked, an iteration runs, and the dense gradients end up reduced."""
    from tests.dist_utils import run_distributed
    res = run_distributed(_parallel_sizes_worker, 2, flags)
    for r in res:
        assert (r["dp"], r["cp"], r["ep"]) == (dp, cp, cp)
        assert r["gnorm"] > 0
    # sequence parallelism splits the preset's sequence over the group; replicas see all of it
    from fluidmoe_b200.tools.model_configs import get_model_config
    seq = int(get_model_config("tiny_test")["seq_len"])
    assert res[0]["rows"] == res[1]["rows"] == seq // cp
