"""The training examples: token cache, the training script on a token file (one CPU process, two
micro-batches per step, save and resume), the shared harness around a foreign block stack, and the
comparison driver's table."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "examples"))

TINY = ["--layers", "1", "--hidden", "64", "--heads", "4", "--kv-heads", "2", "--ffn", "96", "--experts", "4",
        "--vocab", "300", "--seq", "32"]


def _corpus(path):
    with open(path, "w", encoding="utf-8") as f:
        for d in range(6):
            f.write(f" = Article {d} = \n\n")
            f.write(" ".join(f"word{(d * 7 + i) % 23}" for i in range(200)) + " \n\n")
    return path


def test_token_cache_and_dataset(tmp_path):
    import text_dataset as td
    text = _corpus(str(tmp_path / "corpus.txt"))
    out = td.build_token_cache(text, str(tmp_path / "tokens.bin"))
    toks = np.fromfile(out, dtype=np.uint16)
    assert (toks == td.BYTE_EOD).sum() == 6 and toks.max() <= 256        # one end-of-document id per article
    stamp = os.path.getmtime(out)
    assert td.build_token_cache(text, out) == out and os.path.getmtime(out) == stamp      # cache is reused
    ds = td.TokenFileDataset(out, 65)
    assert len(ds) == (len(toks) - 1) // 65 and ds[0].shape == (65,) and ds[0].dtype == torch.int64
    assert torch.equal(ds[len(ds)], ds[0])
    td.main(["--text", text, "--out", str(tmp_path / "again.bin")])
    assert np.array_equal(np.fromfile(str(tmp_path / "again.bin"), dtype=np.uint16), toks)


def test_pretrain_script_trains_saves_and_resumes(tmp_path, capsys):
    import text_dataset as td
    import pretrain_fluidmoe
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler
    data = td.build_token_cache(_corpus(str(tmp_path / "c.txt")), str(tmp_path / "t.bin"))
    BackwardScheduler.reset()
    pretrain_fluidmoe.main(TINY + ["--steps", "4", "--micro-batches", "2", "--data", data, "--lr", "1e-2",
                                   "--save", str(tmp_path / "ck")])
    lines = [l for l in capsys.readouterr().out.splitlines() if "lm loss" in l]
    assert len(lines) == 4 and "grad norm" in lines[0]
    losses = [float(l.split("lm loss:")[1].split("|")[0]) for l in lines]
    assert losses[-1] < losses[0]
    assert os.path.exists(tmp_path / "ck" / "manifest.json")
    BackwardScheduler.reset()
    pretrain_fluidmoe.main(TINY + ["--steps", "1", "--data", data, "--load", str(tmp_path / "ck"), "--mode", "F"])
    resumed = [l for l in capsys.readouterr().out.splitlines() if "lm loss" in l]
    assert float(resumed[0].split("lm loss:")[1].split("|")[0]) < losses[0]       # starts from the trained weights
    BackwardScheduler.reset()


def test_baseline_loop_trains_a_foreign_block_stack(capsys, monkeypatch):
    """The loop the Megatron / DeepSpeed arms use, around a plain torch block stack."""
    import _baseline_loop as loop
    monkeypatch.setattr(sys, "argv", ["x"] + TINY + ["--steps", "3", "--lr", "1e-2"])
    args = loop.parse()

    def build_blocks(cfg, pc, device):
        assert cfg["ffn_hidden"] == 96 and cfg["norm_type"] == "layernorm"
        return torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.GELU(), torch.nn.Linear(64, 64))
    loop.train(args, build_blocks, arm="stub")
    lines = [l for l in capsys.readouterr().out.splitlines() if "lm loss" in l]
    assert len(lines) == 3 and "grad norm" in lines[-1]


def test_external_arm_scripts_report_missing_packages():
    for script in ("pretrain_megatron.py", "pretrain_deepspeed.py"):
        res = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), "--steps", "1"],
                             capture_output=True, text=True, timeout=300, cwd=ROOT)
        assert res.returncode == 0 and "baseline unavailable" in res.stdout, res.stdout + res.stderr


@pytest.mark.skipif(torch.cuda.is_available(), reason="CPU-sized run of the driver")
def test_run_training_driver_prints_the_comparison_table(tmp_path):
    env = dict(os.environ, NGPU="1", STEPS="3", LAYERS="1", HIDDEN="64", HEADS="4", KV="2", FFN="96", EXPERTS="4",
               SEQ="32", VOCAB="300", OUT=str(tmp_path / "logs"))
    res = subprocess.run(["bash", os.path.join(ROOT, "examples", "run_training.sh")], capture_output=True,
                         text=True, timeout=900, cwd=ROOT, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    table = res.stdout
    assert "final lm loss" in table and "fluidmoe_full" in table and "fluidmoe_baseline" in table
    assert "megatron" in table and "baseline unavailable" in table
