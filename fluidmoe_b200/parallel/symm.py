"""Symmetric memory: one slab of device memory per rank, mapped into every peer over NVLink.

``SymmetricHeap`` hands out tensors that live at the same offset in every rank's slab, together
with a device table of the peers' addresses, which is what the fused kernels take to store into
(or load from) another GPU.  Allocation is collective by convention: every rank performs the
same sequence of ``alloc`` calls, so offsets agree without communication.  Tensors returned are
non-owning views; ``reset()``/``close()`` release the slab for everyone.

This replaces the reference's NVSHMEM symmetric heap (fluid/csrc/nvshmem_ops.cpp:119-177,
fluid/core/p2p_backend.py:187-260) with plain CUDA IPC mappings and kernels of this library.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _native
from ..ops.gemm import status_buffer

_ALIGN = 1024


class _RawCudaBuffer:
    """Object exposing ``__cuda_array_interface__`` for a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self._owner = owner
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def tensor_from_ptr(ptr: int, nbytes: int, device, owner=None) -> torch.Tensor:
    """uint8 tensor over ``nbytes`` of device memory at ``ptr`` (non-owning)."""
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes, owner), device=device)


@dataclass
class SymmTensor:
    """A tensor that exists at the same slab offset on every rank of the heap's group."""

    local: torch.Tensor            # this rank's instance
    offset: int                    # byte offset inside the slab
    peer_addrs: List[int]          # address of the instance of every rank (index = group rank)
    peer_table: torch.Tensor       # int64 device tensor of ``peer_addrs`` (a ``T* const*`` for kernels)

    @property
    def ptr_table(self) -> int:
        return self.peer_table.data_ptr()


_CANARY_BYTE = 0xC5


class SymmetricHeap:
    def __init__(self, group=None, nbytes: int = 1 << 30, device=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.nbytes = int(math.ceil(nbytes / _ALIGN) * _ALIGN)
        lib = _native.lib()
        with torch.cuda.device(self.device):
            self._base, handle = lib.symm_alloc(self.nbytes)
        self._peer_bases: List[int] = [0] * self.world
        self._peer_bases[self.rank] = self._base
        if self.world > 1:
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            with torch.cuda.device(self.device):
                for r, h in enumerate(handles):
                    if r != self.rank:
                        self._peer_bases[r] = lib.symm_open(h)
        self._slab = tensor_from_ptr(self._base, self.nbytes, self.device, owner=self)
        self._cursor = 0
        self._high_water = 0     # the slab is zero-filled at creation; bytes above this mark are still zero
        self._closed = False
        # Debug aid (FLUIDMOE_SYMM_CANARY=1): a guard block filled with a byte pattern follows every
        # allocation; ``check_canaries()`` tells which buffer a kernel (local or a peer's) overran.
        import os
        self._canary = os.environ.get("FLUIDMOE_SYMM_CANARY", "0") == "1"
        self._guards: List[tuple] = []     # (start of guard, label)
        self._barrier_flags = self.alloc((max(self.world, 1),), torch.int32)
        self._barrier_epoch = 0
        self._marks: List[int] = []

    # ------------------------------------------------------------------ allocation
    def alloc(self, shape: Sequence[int], dtype: torch.dtype, zero: bool = True) -> SymmTensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        start = self._cursor
        end = start + int(math.ceil(max(nbytes, 1) / _ALIGN) * _ALIGN)
        data_end = end
        if self._canary:
            end += _ALIGN
        if end > self.nbytes:
            raise MemoryError(
                f"symmetric heap exhausted: need {end - start} more bytes, {self.nbytes - start} left")
        self._cursor = end
        if self._canary:
            self._slab[data_end:end].fill_(_CANARY_BYTE)
            self._guards = [g for g in self._guards if g[0] < start]     # guards of released regions
            self._guards.append((data_end, f"allocation at byte {start} ({tuple(shape)} {dtype})"))
        # A tensor of its own over the slice (not a view of the slab): every allocation gets its
        # own autograd version counter, so an in-place update of one buffer (a counter reset, an
        # in-place RoPE) does not invalidate tensors saved for backward that live in another.
        local = tensor_from_ptr(self._base + start, max(nbytes, 1), self.device, owner=self)[:nbytes] \
            .view(dtype).view(*shape)
        if zero and start < self._high_water:
            # Re-used region: clear it.  Peers may only write here after the next collective
            # synchronisation of the group (callers that hand the buffer to peers do that).
            local.zero_()
        self._high_water = max(self._high_water, end)
        addrs = [b + start for b in self._peer_bases]
        table = torch.tensor(addrs, dtype=torch.int64, device=self.device)
        return SymmTensor(local, start, addrs, table)

    def check_canaries(self) -> None:
        """Host-synchronising check of every guard block; raises ``RuntimeError`` naming the first
        allocation whose guard was overwritten.  No-op unless the heap was created with
        ``FLUIDMOE_SYMM_CANARY=1``."""
        if not self._canary:
            return
        for gstart, label in self._guards:
            if gstart >= self._cursor:
                continue
            block = self._slab[gstart:gstart + _ALIGN]
            if not bool((block == _CANARY_BYTE).all().item()):
                bad = int((block != _CANARY_BYTE).nonzero()[0].item())
                raise RuntimeError(f"symmetric heap guard overwritten {bad} bytes past the end of {label} "
                                   f"on rank {self.rank}")

    def mark(self) -> None:
        self._marks.append(self._cursor)

    def release_to_mark(self) -> None:
        """Return everything allocated since the matching ``mark()`` (collective by convention)."""
        self._cursor = self._marks.pop()

    @property
    def bytes_used(self) -> int:
        return self._cursor

    # ------------------------------------------------------------------ primitives
    def barrier(self, timeout_ms: float = 4000.0) -> None:
        """Stream-ordered barrier over the group, executed by a kernel (no host sync)."""
        self._barrier_epoch += 1
        if self.world == 1:
            return
        _native.lib().symm_barrier(
            self._barrier_flags.ptr_table, self.rank, self.world, self._barrier_epoch,
            int(timeout_ms * 1e6), status_buffer(self.device).data_ptr(), _native.stream_ptr())

    def sync_group(self) -> None:
        """Host-side rendezvous: every rank has finished its allocations (and clears) before any
        rank lets a kernel write into a peer."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        lib = _native.lib()
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        for r, b in enumerate(self._peer_bases):
            if r != self.rank and b:
                lib.symm_close(b)
        if self.world > 1:
            dist.barrier(group=self.group)
        lib.symm_free(self._base)


class SymmAllToAll:
    """Device-initiated all-to-all (unfused): each rank stores its slices straight into its
    peers' receive buffers and publishes them with a flag; receivers poll with a time limit.

    Equal splits of at most ``max_bytes_per_peer`` bytes per peer.  The receive buffer is double
    buffered so that a peer may start the next exchange before this rank consumed the last.
    """

    def __init__(self, heap: SymmetricHeap, max_bytes_per_peer: int, num_ctas: int = 32):
        self.heap = heap
        P = heap.world
        self.P = P
        self.cap = int(math.ceil(max_bytes_per_peer / 16) * 16)
        self.recv = [heap.alloc((P * self.cap,), torch.uint8, zero=False) for _ in range(2)]
        self.flags = [heap.alloc((P,), torch.int32) for _ in range(2)]
        self.counters = torch.zeros(P, dtype=torch.int32, device=heap.device)
        self.epoch = 0
        self.num_ctas = num_ctas
        dev = heap.device
        self._dst_offs = torch.full((P,), heap.rank * self.cap, dtype=torch.int64, device=dev)
        self._cache: Dict[int, tuple] = {}
        heap.sync_group()

    def __call__(self, x: torch.Tensor, timeout_ms: float = 4000.0) -> torch.Tensor:
        P, heap = self.P, self.heap
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        assert nbytes % P == 0
        per = nbytes // P
        assert per % 16 == 0 and per <= self.cap, (per, self.cap)
        self.epoch += 1
        slot = self.epoch & 1
        if per not in self._cache:
            dev = heap.device
            self._cache[per] = (
                torch.arange(P, dtype=torch.int64, device=dev) * per,
                torch.full((P,), per, dtype=torch.int64, device=dev),
            )
        send_offs, send_bytes = self._cache[per]
        lib = _native.lib()
        gen = (self.epoch + 1) // 2
        lib.a2a_push(x.data_ptr(), send_offs.data_ptr(), send_bytes.data_ptr(),
                     self.recv[slot].ptr_table, self._dst_offs.data_ptr(), self.flags[slot].ptr_table,
                     self.counters.data_ptr(), heap.rank, P, gen, self.num_ctas, _native.stream_ptr())
        lib.a2a_wait(self.flags[slot].local.data_ptr(), heap.rank, P, gen, int(timeout_ms * 1e6),
                     status_buffer(heap.device).data_ptr(), _native.stream_ptr())
        out = self.recv[slot].local.view(P, self.cap)[:, :per]
        return out.reshape(-1).view(x.dtype).view(x.shape)


class SymmAllReduce:
    """Two-shot sum all-reduce over peer memory on a symmetric buffer (in place)."""

    def __init__(self, heap: SymmetricHeap, numel: int, dtype: torch.dtype, num_ctas: int = 32):
        assert dtype in (torch.float32, torch.bfloat16)
        self.heap = heap
        self.buf = heap.alloc((numel,), dtype)
        self.flags = heap.alloc((heap.world + 2,), torch.int32)
        self.epoch = 0
        self.num_ctas = num_ctas  # fixed for the life of the object (grid-wide hand-off counts CTAs)
        heap.sync_group()

    def __call__(self, numel: Optional[int] = None, scale: float = 1.0, timeout_ms: float = 4000.0) -> torch.Tensor:
        heap = self.heap
        n = self.buf.local.numel() if numel is None else numel
        if heap.world == 1:
            if scale != 1.0:
                self.buf.local[:n].mul_(scale)
            return self.buf.local
        self.epoch += 1
        _native.lib().allreduce_p2p(
            self.buf.ptr_table, n, int(self.buf.local.dtype == torch.float32), float(scale),
            self.flags.ptr_table, heap.rank, heap.world, self.epoch, self.num_ctas,
            int(timeout_ms * 1e6), status_buffer(heap.device).data_ptr(), _native.stream_ptr())
        return self.buf.local


class SymmGradReducer:
    """Flat gradient buffers in symmetric memory, reduced slice by slice by the two-shot kernel.

    ``allocator(n, dtype)`` has the signature ``FlatGradBuffer.setup`` takes and returns this rank's
    instance of a symmetric buffer; ``reduce(chunk, pre_scale)`` has the signature of the
    scheduler's reduce functions: ``chunk`` must be a slice of a buffer handed out by the allocator.
    Every rank reads the peers' copies of its 1/P of the slice over NVLink, adds, scales and writes
    the result into every copy (``fm_allreduce_p2p_slice``), so the pre-scale of the average costs
    nothing extra.  A slice that does not start on a 16-byte boundary, or a group other than the
    heap's, goes through ``fallback`` (the library collective).  This is the counterpart of the
    NCCL all-reduce the reference trickles into its communication gaps
    (fluid/core/scheduler.py:553-695)."""

    def __init__(self, heap: SymmetricHeap, fallback=None, num_ctas: int = 24, timeout_ms: float = 8000.0):
        self.heap = heap
        self.fallback = fallback
        self.num_ctas = num_ctas
        self.timeout_ns = int(timeout_ms * 1e6)
        self._bufs: List[SymmTensor] = []
        self.flags = heap.alloc((heap.world + 2,), torch.int32)
        self.epoch = 0
        self.calls = 0
        self.fallback_calls = 0

    def allocator(self, n: int, dtype: torch.dtype) -> torch.Tensor:
        t = self.heap.alloc((max(int(n), 4),), dtype)
        self._bufs.append(t)
        return t.local[:n]

    def _locate(self, chunk: torch.Tensor):
        addr = chunk.data_ptr()
        for t in self._bufs:
            lo = t.local.data_ptr()
            if lo <= addr < lo + t.local.numel() * t.local.element_size():
                return t, (addr - lo) // t.local.element_size()
        return None, 0

    def reduce(self, chunk: torch.Tensor, pre_scale: float = 1.0) -> None:
        heap = self.heap
        if heap.world == 1:
            if pre_scale != 1.0:
                chunk.mul_(pre_scale)
            return
        t, off = self._locate(chunk)
        ok = t is not None and chunk.is_contiguous() and (off * chunk.element_size()) % 16 == 0 \
            and chunk.dtype in (torch.float32, torch.bfloat16)
        if not ok:
            self.fallback_calls += 1
            if self.fallback is None:
                raise ValueError("gradient slice is not in a symmetric buffer (or not 16-byte aligned) and no "
                                 "fallback reduce function was given")
            self.fallback(chunk, pre_scale)
            return
        self.epoch += 1
        self.calls += 1
        _native.lib().allreduce_p2p_slice(
            t.ptr_table, int(off), chunk.numel(), int(chunk.dtype == torch.float32), float(pre_scale),
            self.flags.ptr_table, heap.rank, heap.world, self.epoch, self.num_ctas, self.timeout_ns,
            status_buffer(heap.device).data_ptr(), _native.stream_ptr())


class NvlsAllReduce:
    """In-switch (NVLS) sum all-reduce on an fp32 buffer (in place).

    The buffer comes from PyTorch's VMM-based symmetric allocator, which binds every rank's copy to
    one NVLink multicast object and hands back the multicast address; the reduction itself is this
    library's kernel (``multimem.ld_reduce`` / ``multimem.st``, one slice per rank) bracketed by the
    bounded peer barrier of the two-shot kernel.  ``available`` is False when the allocator or the
    multicast mapping is missing (no NVSwitch, unsupported driver); callers then use
    ``SymmAllReduce`` or the library collective.  Counterpart of the reference's reliance on NCCL's
    all-reduce for the trickled gradient reduction (fluid/core/scheduler.py:188-213).

    Not to be used in tests that let a rank leave while peers keep running: a rank that exits
    while its memory is bound to a multicast object can fault the other ranks' GPUs.
    """

    def __init__(self, heap: SymmetricHeap, numel: int, group=None, num_ctas: int = 0):
        self.heap = heap
        self.numel = numel
        self.num_ctas = num_ctas
        self.epoch = 0
        self.available = False
        self.local = None
        self._mc_ptr = 0
        if heap.world <= 1 or heap.device.type != "cuda":
            return
        try:
            import torch.distributed._symmetric_memory as symm_mem
            g = group if group is not None else dist.group.WORLD
            self.local = symm_mem.empty(numel, dtype=torch.float32, device=heap.device)
            self._handle = symm_mem.rendezvous(self.local, g.group_name)
            self._mc_ptr = int(getattr(self._handle, "multicast_ptr", 0) or 0)
        except Exception:  # noqa: BLE001 - allocator / multicast unsupported on this system
            self._mc_ptr = 0
        self.available = self._mc_ptr != 0
        if self.available:
            self.flags = heap.alloc((heap.world + 2,), torch.int32)
            heap.sync_group()

    def __call__(self, numel: Optional[int] = None, scale: float = 1.0, timeout_ms: float = 4000.0) -> torch.Tensor:
        if not self.available:
            raise RuntimeError("NVLS all-reduce is not available on this system")
        n = self.numel if numel is None else numel
        self.epoch += 1
        _native.lib().allreduce_nvls(self._mc_ptr, n, float(scale), self.flags.ptr_table, self.heap.rank,
                                     self.heap.world, self.epoch, self.num_ctas, int(timeout_ms * 1e6),
                                     status_buffer(self.heap.device).data_ptr(), _native.stream_ptr())
        return self.local
