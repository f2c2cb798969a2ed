"""Parity with the reference implementation on its own architecture (GELU experts, LayerNorm,
padded capacity): same weights through ``load_reference_state_dict``, same inputs; output, input
gradient, every parameter gradient and a 20-step loss curve.  Needs the reference installed under
``baseline/_ref`` (see ``fluidmoe_b200/tools/parity_reference.py``).

There is no one-GPU case: with an expert-parallel group of one rank the reference never runs its
local expert FFN (the local FC1 call sits inside its per-partner loop, fluid/moe/forward.py:690-728,
which has no iterations, so ``local_act`` stays None and ``combined_output`` is never written,
fluid/moe/forward.py:1045-1051) and its layer returns the attention half plus the stale contents of
a persistent buffer.  Parity is therefore defined from two ranks up."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world: int, port: int, extra=()):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "fluidmoe_b200.tools.parity_reference",
           "--steps", "8", *extra]
    res = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=900)
    lines = [l for l in res.stdout.splitlines() if l.startswith("PARITY_RESULT ")]
    assert res.returncode == 0 and lines, res.stdout[-3000:] + res.stderr[-3000:]
    return json.loads(lines[-1][len("PARITY_RESULT "):])


def _need_reference():
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "fluid")):
        pytest.skip("reference not installed under baseline/_ref")


def test_parity_with_reference_two_gpus_fused_transport():
    _need_reference()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    out = _run(2, 29622)
    assert out["ok"] and out["comm"] == "auto", out
    assert out["loss_curve_max_rel"] < 5e-2, out
