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
