"""NVTX ranges, active only when ``FLUID_NVTX=1`` (zero cost otherwise).

Counterpart of fluid/core/nvtx.py:23-56 of the reference.
"""
from __future__ import annotations

import contextlib
import os

import torch

ENABLED = os.environ.get("FLUID_NVTX", "0") == "1"


def _active() -> bool:
    return ENABLED and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    if _active():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def nvtx_range_push(name: str) -> None:
    if _active():
        torch.cuda.nvtx.range_push(name)


def nvtx_range_pop() -> None:
    if _active():
        torch.cuda.nvtx.range_pop()
