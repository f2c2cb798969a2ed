"""Train the Megatron-Core baseline block stack with the same loop as ``pretrain_fluidmoe.py``.

    torchrun --nproc-per-node N examples/pretrain_megatron.py --model mixtral_8x7b --steps 20

Needs megatron-core and Transformer Engine (see ``fluidmoe_b200.tools.external_baselines``); exits
with a one-line message when they are not installed.  The reference keeps the same comparison arm
(examples/pretrain_megatron.py:32-172).
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from examples._baseline_loop import run  # noqa: E402

if __name__ == "__main__":
    run("megatron")
