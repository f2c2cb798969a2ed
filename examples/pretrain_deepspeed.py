"""Train the DeepSpeed (Ulysses attention + DeepSpeed MoE) baseline block stack.

    torchrun --nproc-per-node N examples/pretrain_deepspeed.py --model mixtral_8x7b --steps 20

Needs deepspeed (see ``fluidmoe_b200.tools.external_baselines``); exits with a one-line message when
it is not installed.  The reference's arm runs its blocks on a DeepSpeed ZeRO-0 engine
(examples/pretrain_deepspeed.py:67-369); here the blocks are trained by the same plain loop as the
other arms, with gradients all-reduced in fp32.
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from examples._baseline_loop import run  # noqa: E402

if __name__ == "__main__":
    run("deepspeed")
