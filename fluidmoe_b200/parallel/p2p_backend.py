"""Pairwise exchange back-ends for the round-ordered forward overlap path.

``exchange`` is stream-ordered: it is issued on the communication stream and the caller waits on
the event it records before consuming the received data.

* ``CollectiveP2PBackend``: ``torch.distributed`` isend/irecv pairs (NCCL on GPUs, gloo on CPU).
* ``SymmetricP2PBackend``: a kernel of this library stores the payload into the partner's
  symmetric receive buffer over NVLink and raises a flag; the receiver polls it with a time
  limit.  Flags are kept per process group so that the attention and expert groups never
  observe each other's counters.

Selection follows ``FLUIDMOE_P2P_BACKEND`` = ``nccl`` | ``symm`` (alias ``nvshmem``) | ``auto``.
Counterpart of fluid/core/p2p_backend.py:55-468 of the reference.
"""
from __future__ import annotations

import os
import threading
import warnings
from abc import ABC, abstractmethod
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native
from .streams import on_stream


class P2PBackend(ABC):
    @abstractmethod
    def exchange(self, send_buf, recv_buf, partner_global_rank: int, partner_local_rank: int,
                 group, comm_stream, event) -> None:
        """Send ``send_buf`` to and receive ``recv_buf`` from the partner, then record ``event``."""

    @abstractmethod
    def alloc_recv_buffer(self, tag: str, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
        """Return a (cached, grow-only) receive buffer usable with this back-end."""

    @abstractmethod
    def needs_final_wait(self) -> bool: ...

    @abstractmethod
    def final_wait(self) -> None: ...

    def clear_iteration(self) -> None:
        pass

    def finalize(self) -> None:
        pass


class CollectiveP2PBackend(P2PBackend):
    """isend/irecv pairs through ``torch.distributed`` (works for NCCL and gloo groups)."""

    def __init__(self):
        self._reqs = []
        self._bufs: Dict[tuple, torch.Tensor] = {}

    def exchange(self, send_buf, recv_buf, partner_global_rank, partner_local_rank, group,
                 comm_stream, event):
        ops = []
        if recv_buf is not None:
            ops.append(dist.P2POp(dist.irecv, recv_buf, partner_global_rank, group=group))
        if send_buf is not None:
            if send_buf.is_cuda and comm_stream is not None:
                send_buf.record_stream(comm_stream)
            ops.append(dist.P2POp(dist.isend, send_buf, partner_global_rank, group=group))
        if ops:
            with on_stream(comm_stream):
                reqs = dist.batch_isend_irecv(ops)
                if send_buf is not None and not send_buf.is_cuda:
                    for r in reqs:  # gloo: complete now, there is no stream to order against
                        r.wait()
                else:
                    self._reqs.extend(reqs)
                    if reqs:
                        reqs[-1].wait()  # stream-level wait on the communication stream
        if event is not None:
            event.record(comm_stream) if comm_stream is not None else event.record()

    def alloc_recv_buffer(self, tag, numel, dtype, device, group=None):
        device = torch.device(device)
        key = (tag, dtype, device.type, device.index)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < numel:
            buf = torch.empty(max(numel, 1), dtype=dtype, device=device)
            self._bufs[key] = buf
        return buf[:numel]

    def needs_final_wait(self) -> bool:
        return True

    def final_wait(self) -> None:
        if self._reqs:
            self._reqs[-1].wait()

    def clear_iteration(self) -> None:
        self._reqs.clear()


NCCLBackend = CollectiveP2PBackend


class SymmetricP2PBackend(P2PBackend):
    """One-sided put + flag over symmetric memory, issued by a kernel on the comm stream."""

    def __init__(self, heap_bytes: int = 1 << 30):
        from .symm import SymmetricHeap  # noqa: F401 - checked at construction
        self._heap_bytes = heap_bytes
        self._groups: Dict[Tuple, dict] = {}
        self._bufs: Dict[tuple, object] = {}

    def _state(self, group, device):
        from .symm import SymmetricHeap
        # Keyed by the sorted global ranks of the group: stable for the life of the job, unlike
        # id(group), which can be reused after a group object is collected.
        ranks = tuple(dist.get_process_group_ranks(group)) if group is not None else ("world",)
        st = self._groups.get(ranks)
        if st is None:
            heap = SymmetricHeap(group, self._heap_bytes, device)
            P = heap.world
            st = dict(
                heap=heap,
                flags=heap.alloc((P,), torch.int32),
                counters=torch.zeros(P, dtype=torch.int32, device=device),
                sent=[0] * P,       # monotonically increasing per-partner signal values
                zeros64=torch.zeros(P, dtype=torch.int64, device=device),
            )
            self._groups[ranks] = st
        return st

    def alloc_recv_buffer(self, tag, numel, dtype, device, group=None):
        st = self._state(group, torch.device(device))
        key = (tag, dtype, id(st))
        cur = self._bufs.get(key)
        if cur is None or cur.local.numel() < numel:
            cur = st["heap"].alloc((max(numel, 8),), dtype, zero=False)
            self._bufs[key] = cur
        return cur.local[:numel]

    def _locate(self, t: torch.Tensor):
        """Find the symmetric allocation that contains ``t`` and ``t``'s byte offset inside it."""
        addr = t.data_ptr()
        for cur in self._bufs.values():
            lo = cur.local.data_ptr()
            if lo <= addr < lo + cur.local.numel() * cur.local.element_size():
                return cur, addr - lo
        return None, 0

    def exchange(self, send_buf, recv_buf, partner_global_rank, partner_local_rank, group,
                 comm_stream, event):
        if send_buf is None or recv_buf is None:
            raise ValueError("SymmetricP2PBackend.exchange needs both a send and a receive buffer")
        symm, offset = self._locate(recv_buf)
        if symm is None:
            raise ValueError("receive buffer was not allocated by alloc_recv_buffer()")
        assert recv_buf.is_contiguous() and send_buf.is_contiguous()
        st = self._state(group, recv_buf.device)
        heap = st["heap"]
        P, me, q = heap.world, heap.rank, partner_local_rank
        nbytes = send_buf.numel() * send_buf.element_size()
        assert nbytes % 16 == 0, "payload must be a multiple of 16 bytes"
        st["sent"][q] += 1
        epoch = st["sent"][q]
        lib = _native.lib()
        with on_stream(comm_stream):
            s = torch.cuda.current_stream().cuda_stream
            send_buf.record_stream(torch.cuda.current_stream())
            self._push_one(lib, st, send_buf, offset, symm, q, epoch, s)
            lib.wait_flag(st["flags"].local.data_ptr() + 4 * q, epoch, int(4e9),
                          _status(recv_buf.device), s)
            if event is not None:
                event.record(torch.cuda.current_stream())

    def _push_one(self, lib, st, send_buf, offset, symm, q, epoch, stream):
        heap = st["heap"]
        P = heap.world
        # Per-partner flag pointer table: entry p points at rank p's word for *me*; the kernel
        # indexes it as flag_ptrs[p] + my_rank.
        lib.put_signal(send_buf.data_ptr(), send_buf.numel() * send_buf.element_size(),
                       symm.peer_addrs[q] + offset, st["flags"].peer_addrs[q] + 4 * heap.rank, epoch, 16,
                       st["counters"].data_ptr() + 4 * q, stream)

    def needs_final_wait(self) -> bool:
        return False

    def final_wait(self) -> None:
        pass

    def finalize(self) -> None:
        for st in self._groups.values():
            st["heap"].close()
        self._groups.clear()
        self._bufs.clear()


NVSHMEMBackend = SymmetricP2PBackend


def _status(device):
    from ..ops.gemm import status_buffer
    return status_buffer(device).data_ptr()


def _has_peer_access() -> bool:
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        return False
    try:
        return any(torch.cuda.can_device_access_peer(0, j) for j in range(1, torch.cuda.device_count()))
    except Exception:  # noqa: BLE001
        return False


_BACKEND: Optional[P2PBackend] = None
_LOCK = threading.Lock()


def _has_nvlink() -> bool:
    """True when some pair of this machine's GPUs can address each other's memory (what the
    device-initiated transports need; fluid/core/p2p_backend.py:396-407)."""
    if not torch.cuda.is_available():
        return False
    n = torch.cuda.device_count()
    return any(torch.cuda.can_device_access_peer(i, j) for i in range(n) for j in range(i + 1, n))


def get_p2p_backend() -> P2PBackend:
    """Process-wide back-end chosen from ``FLUIDMOE_P2P_BACKEND`` (default ``auto``)."""
    global _BACKEND
    with _LOCK:
        if _BACKEND is not None:
            return _BACKEND
        choice = os.environ.get("FLUIDMOE_P2P_BACKEND", "auto").lower()
        if choice in ("symm", "nvshmem"):
            _BACKEND = SymmetricP2PBackend()
        elif choice == "nccl" or choice == "gloo":
            _BACKEND = CollectiveP2PBackend()
        else:
            # auto: the round-ordered pairwise path runs on library point-to-point (NCCL / gloo).
            # Device-initiated transfers are the business of the fused paths
            # (parallel/fused.py); the symmetric pairwise back-end is opt-in.
            _BACKEND = CollectiveP2PBackend()
        return _BACKEND


def reset_p2p_backend() -> None:
    """Drop the process-wide back-end (collective when it owns symmetric memory)."""
    global _BACKEND
    with _LOCK:
        if _BACKEND is not None:
            _BACKEND.finalize()
        _BACKEND = None
