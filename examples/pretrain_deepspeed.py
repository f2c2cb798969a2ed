"""Train the DeepSpeed arm (Ulysses ``DistributedAttention`` + ``deepspeed.moe.layer.MoE`` blocks)
with the harness, data and log format of ``pretrain_fluidmoe.py``.

    torchrun --nproc-per-node N examples/pretrain_deepspeed.py --layers 4 --steps 100 [--engine]

With ``--engine`` the model is handed to ``deepspeed.initialize`` with a ZeRO-0 configuration and
fp32 gradient communication, which is how the reference runs this arm
(examples/pretrain_deepspeed.py:67-369, ZeRO stage 0 at :275); without it the blocks are trained by
the plain loop of the other arms with gradients all-reduced in fp32.  Needs deepspeed: without it
the script prints one line and exits.
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import _baseline_loop as loop  # noqa: E402
from fluidmoe_b200.tools import external_baselines as eb  # noqa: E402
from fluidmoe_b200.tools.experiment_configs import get_deepspeed_ulysses_defaults  # noqa: E402


def build_blocks(cfg, pc, device):
    eb._need("deepspeed")
    return eb.build_deepspeed_ulysses_baseline(cfg, pc.cp_group, max(1, pc.world_size), device=device)


def deepspeed_config(args) -> dict:
    """ZeRO-0, bf16 parameters, fp32 gradient reduction, AdamW: the reference's settings for this arm."""
    return {
        "train_micro_batch_size_per_gpu": args.batch,
        "gradient_accumulation_steps": 1,
        "zero_optimization": {"stage": int(get_deepspeed_ulysses_defaults()["zero_stage"])},
        "bf16": {"enabled": True},
        "communication_data_type": "fp32",
        "optimizer": {"type": "AdamW", "params": {"lr": args.lr, "weight_decay": 0.0, "betas": [0.9, 0.999]}},
        "steps_per_print": 10 ** 9,
    }


def wrap_engine(model, args):
    import deepspeed
    engine, _, _, _ = deepspeed.initialize(model=model, model_parameters=[p for p in model.parameters()],
                                           config=deepspeed_config(args))

    def step(loss):
        engine.backward(loss)
        engine.step()
    return engine, step


def _extra(ap):
    ap.add_argument("--engine", action="store_true", help="train through deepspeed.initialize (ZeRO-0)")


if __name__ == "__main__":
    a = loop.parse(_extra)
    loop.train(a, build_blocks, wrap_engine if a.engine else None, arm="deepspeed")
