"""Streams and events shared by forward overlap, the backward scheduler and the all-reduce.

One side stream carries every collective (all-to-all *and* gradient all-reduce, which therefore
never run concurrently), a second one carries deferred weight-gradient GEMMs when they are asked
to run beside a communication kernel.  On CPU tensors (the gloo test path) streams and events are
replaced by no-op stand-ins so that the scheduling logic is exercised unchanged.

Counterpart of the reference's StreamManager (fluid/core/stream.py:18-107).
"""
from __future__ import annotations

import contextlib
import threading
from typing import Dict, Hashable, Optional

import torch


class NullEvent:
    """Stand-in for torch.cuda.Event on CPU: work is synchronous, so every event is complete."""

    def __init__(self, enable_timing: bool = False):
        import time

        self._t = None
        self._time = time

    def record(self, stream=None):
        self._t = self._time.perf_counter()

    def wait(self, stream=None):
        pass

    def synchronize(self):
        pass

    def query(self) -> bool:
        return True

    def elapsed_time(self, other: "NullEvent") -> float:
        if self._t is None or other._t is None:
            return 0.0
        return (other._t - self._t) * 1e3


class NullStream:
    """Stand-in for torch.cuda.Stream on CPU."""

    def wait_event(self, event):
        pass

    def wait_stream(self, stream):
        pass

    def synchronize(self):
        pass

    def record_event(self, event=None):
        event = event or NullEvent()
        event.record()
        return event


def is_cuda_device(device) -> bool:
    return torch.device(device).type == "cuda"


def make_event(device, enable_timing: bool = False):
    return torch.cuda.Event(enable_timing=enable_timing) if is_cuda_device(device) else NullEvent()


def current_stream(device):
    return torch.cuda.current_stream(device) if is_cuda_device(device) else NullStream()


@contextlib.contextmanager
def on_stream(stream):
    """``with on_stream(s):`` works for CUDA streams and for the CPU stand-in."""
    if isinstance(stream, NullStream) or stream is None:
        yield
    else:
        with torch.cuda.stream(stream):
            yield


class StreamManager:
    """Process-wide owner of the side streams and of a keyed pool of reusable events."""

    def __init__(self):
        self._device: Optional[torch.device] = None
        self._comm = None
        self._dw = None
        self._ar = None
        self._events: Dict[Hashable, object] = {}
        self._lock = threading.Lock()
        self.data_ready_event = None
        self._one_sided_ready = False

    def initialize(self, device) -> None:
        device = torch.device(device)
        with self._lock:
            if self._device is not None:
                if self._device != device:
                    raise RuntimeError(
                        f"StreamManager already bound to {self._device}; cannot rebind to {device}")
                return
            self._device = device
            if device.type == "cuda":
                # Collectives at high priority so that they are issued ahead of queued compute.
                lo, hi = torch.cuda.Stream.priority_range()
                self._comm = torch.cuda.Stream(device=device, priority=hi)
                self._ar = self._comm  # all-reduce shares the collective stream by design
                self._dw = torch.cuda.Stream(device=device, priority=lo)
            else:
                self._comm = NullStream()
                self._ar = self._comm
                self._dw = NullStream()
            self.data_ready_event = make_event(device)

    @property
    def initialized(self) -> bool:
        return self._device is not None

    @property
    def device(self):
        return self._device

    @property
    def comm_stream(self):
        return self._comm

    @property
    def ar_stream(self):
        return self._ar

    @property
    def dw_stream(self):
        return self._dw

    def get_sync_event(self, key: Hashable, enable_timing: bool = False):
        ev = self._events.get(key)
        if ev is None:
            ev = make_event(self._device, enable_timing)
            self._events[key] = ev
        return ev

    def init_nvshmem(self) -> None:
        """Bring up the one-sided transport of the pairwise back-end.  The reference initialises
        NVSHMEM here (fluid/core/stream.py:109-176); its place is taken by the symmetric heap
        over peer memory, which the symmetric back-end maps for the world group.  With the
        collective back-end selected there is nothing to bring up and the flag stays False."""
        if self._one_sided_ready:
            return
        if self._device is None or self._device.type != "cuda":
            raise RuntimeError("the one-sided transport needs a CUDA device: call initialize(device) first")
        from .p2p_backend import SymmetricP2PBackend, get_p2p_backend
        backend = get_p2p_backend()
        if isinstance(backend, SymmetricP2PBackend):
            backend._state(None, self._device)
            self._one_sided_ready = True

    @property
    def nvshmem_initialized(self) -> bool:
        return self._one_sided_ready

    def reset(self) -> None:
        with self._lock:
            self._one_sided_ready = False
            self._device = None
            self._comm = self._dw = self._ar = None
            self._events.clear()
            self.data_ready_event = None


# One manager per device type: a process drives one GPU, but CPU-resident models (tests, the
# gloo path) may live beside it and must not share its streams.
_MANAGERS = {"cpu": StreamManager(), "cuda": StreamManager()}


def get_stream_manager(device=None) -> StreamManager:
    """Manager for ``device`` (by type).  Without a device: the CUDA manager once it is bound,
    else the CPU manager once it is bound, else the one matching the machine."""
    if device is not None:
        return _MANAGERS[torch.device(device).type if torch.device(device).type == "cuda" else "cpu"]
    if _MANAGERS["cuda"].initialized:
        return _MANAGERS["cuda"]
    if _MANAGERS["cpu"].initialized:
        return _MANAGERS["cpu"]
    return _MANAGERS["cuda" if torch.cuda.is_available() else "cpu"]
