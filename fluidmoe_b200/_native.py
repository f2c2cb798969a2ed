"""Loader of the in-tree native library (``fluidmoe_b200/_C*.so``).

On a machine with a GPU the CUDA kernels are the only implementation of the hot ops, so a
missing library is an error there; on a CPU-only machine the pure-PyTorch reference path is
used instead and ``available()`` is False.
"""
from __future__ import annotations

import importlib

import torch

_C = None
_ERR = None


def _try_load():
    global _C, _ERR
    if _C is not None or _ERR is not None:
        return
    try:
        _C = importlib.import_module("fluidmoe_b200._C")
    except Exception as e:  # noqa: BLE001 - recorded and re-raised by lib()
        _ERR = e


def available() -> bool:
    """True when the native library is importable *and* a CUDA device is present."""
    _try_load()
    return _C is not None and torch.cuda.is_available()


def lib():
    """Return the extension module; raise loudly when it cannot be loaded."""
    _try_load()
    if _C is None:
        raise RuntimeError(
            "fluidmoe_b200 native library is not built (run `python -m fluidmoe_b200.build`): "
            f"{_ERR!r}"
        )
    return _C


def use_native(*tensors) -> bool:
    """Decide the code path for an op: CUDA tensors -> native kernels (mandatory), CPU -> torch."""
    if not tensors or not all(t.is_cuda for t in tensors if t is not None):
        return False
    lib()  # raises if missing: never fall back silently on a GPU box
    return True


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream
