"""Benchmark / tuner defaults and their persistence.

The reference keeps tuned values by rewriting its own Python source
(tools/experiment_configs.py:64-83).  Here tuned values live in a JSON file next to this module
(``tuned_defaults.json``, or the path in ``FLUIDMOE_TUNED_DEFAULTS``); the code is never edited.
"""
from __future__ import annotations

import json
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))

BLOCK_BENCHMARK_DEFAULTS = dict(
    dp_size=1, cp_size=2, ep_size=2,
    moe_combine_chunks=2, moe_dispatch_chunks=2, attn_proj_chunks=8, attn_qkv_chunks=4,
    warmup=10, iters=50,
    gap_budgets=dict(moe_combine=0.5, moe_dispatch=0.5, attn_proj=0.3, attn_qkv=0.3),
    shared_ar_bw=3.0e8,   # bytes / ms; NVLink-class default, replaced by the tuner's measurement
    expert_ar_bw=3.0e8,
)
TUNE_DEFAULTS = dict(max_chunks=8, min_saving_ms=0.05, warmup=3, iters=10, ar_sizes_mb=(1, 4, 16, 64, 256, 512),
                     gap_percentile=10, gap_safety=0.8)
# settings of the DeepSpeed-Ulysses comparison arm (examples/pretrain_deepspeed.py, tools/external_baselines.py)
DEEPSPEED_ULYSSES_DEFAULTS = dict(zero_stage=0, learning_rate=1e-4, warmup=3, iters=10)


def get_tune_defaults() -> dict:
    """A copy of the tuner's settings (tools/experiment_configs.py:56-57 of the reference)."""
    return json.loads(json.dumps(TUNE_DEFAULTS))


def get_deepspeed_ulysses_defaults() -> dict:
    return dict(DEEPSPEED_ULYSSES_DEFAULTS)


def _path() -> str:
    return os.environ.get("FLUIDMOE_TUNED_DEFAULTS", os.path.join(_HERE, "tuned_defaults.json"))


def get_block_benchmark_defaults(node: Optional[str] = None) -> dict:
    """Defaults merged with persisted tuned values (optionally those of a named node)."""
    cfg = json.loads(json.dumps(BLOCK_BENCHMARK_DEFAULTS))
    try:
        with open(_path()) as f:
            saved = json.load(f)
    except (OSError, ValueError):
        return cfg
    entry = saved.get(node or "default", saved.get("default", {}))
    for k, v in entry.items():
        if isinstance(v, dict) and isinstance(cfg.get(k), dict):
            cfg[k].update(v)
        else:
            cfg[k] = v
    return cfg


def persist_block_benchmark_defaults(values: dict, node: Optional[str] = None) -> str:
    """Merge ``values`` into the persisted defaults (of ``node``) and return the file path."""
    path = _path()
    try:
        with open(path) as f:
            saved = json.load(f)
    except (OSError, ValueError):
        saved = {}
    saved.setdefault(node or "default", {}).update(values)
    with open(path, "w") as f:
        json.dump(saved, f, indent=1, sort_keys=True)
    return path
