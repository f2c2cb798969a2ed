"""Train a Megatron-Core MoE block stack (the comparison arm) with the harness, data and log format
of ``pretrain_fluidmoe.py``.

    torchrun --nproc-per-node N examples/pretrain_megatron.py --layers 4 --steps 100

The blocks come from Megatron-Core's Transformer-Engine layer spec with the all-to-all token
dispatcher, padded expert capacity, grouped GEMM and all-to-all context parallelism over the whole
group (``fluidmoe_b200.tools.external_baselines.build_megatron_baseline``), i.e. the configuration
of the reference's baseline (tools/megatron_baseline.py:118-160).  The reference runs this arm
through Megatron's ``pretrain()`` (examples/pretrain_megatron.py:32-172); here the stack is trained
by the plain loop the other arms use, so that the three logs differ in the blocks only.  Needs
megatron-core and Transformer Engine: without them the script prints one line and exits.
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import _baseline_loop as loop  # noqa: E402
from fluidmoe_b200.tools import external_baselines as eb  # noqa: E402


def _init_megatron_parallel_state(world: int) -> None:
    """Megatron-Core layers look their process groups up in ``parallel_state``."""
    from megatron.core import parallel_state as mpu
    if not mpu.model_parallel_is_initialized():
        mpu.initialize_model_parallel(tensor_model_parallel_size=1, pipeline_model_parallel_size=1,
                                      context_parallel_size=world, expert_model_parallel_size=world)


def build_blocks(cfg, pc, device):
    eb._need("megatron.core", "transformer_engine")
    _init_megatron_parallel_state(max(1, pc.world_size))
    block = eb.build_megatron_baseline(cfg, pc.cp_group, pc.ep_group, device=device)

    class _Stack(loop.torch.nn.Module):        # TransformerBlock takes (hidden_states, attention_mask)
        def __init__(self):
            super().__init__()
            self.block = block

        def forward(self, x):
            return self.block(x, None)
    return _Stack()


if __name__ == "__main__":
    loop.train(loop.parse(), build_blocks, arm="megatron")
