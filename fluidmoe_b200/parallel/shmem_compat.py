"""The entry points of the reference's one-sided extension, served by the symmetric heap.

The reference binds a handful of NVSHMEM calls for its pairwise back-end
(fluid/csrc/nvshmem_ops.cpp:268-289: init / finalize, ``nvshmem_malloc_tensor``, ``nvshmem_ptr``,
``putmem_signal_on_stream``, ``signal_wait_until_on_stream``, ``quiet_on_stream``).  NVSHMEM is not
used here: peer memory is mapped by ``SymmetricHeap`` (CUDA IPC over NVLink), data moves with a
copy kernel that raises a flag with a system-scope release, and a one-thread kernel waits for a
flag with a bounded spin.  This module offers those primitives under the reference's names so
that code written against ``fluid.csrc`` keeps working:

* every rank is a "PE" of the world group; ``nvshmem_init*`` maps one heap for it
  (``FLUIDMOE_SHMEM_HEAP_BYTES``, default 1 GiB).  The unique id of the reference's bootstrap is
  not needed (``torch.distributed`` carries the IPC handles) and is a block of zero bytes;
* allocations come from the heap's bump allocator: ``nvshmem_free_tensor`` forgets the tensor,
  the memory returns when the heap is finalised;
* signals are 32-bit words (``SIGNAL_SET`` stores, ``CMP_GE`` compares); a signal placed in a
  zeroed 64-bit tensor reads the same value up to 2^31 on this little-endian machine;
* ``quiet_on_stream`` has nothing to do: the put kernel's stores are released before its flag.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

_HEAP = None
_ALLOCS: Dict[int, object] = {}      # data_ptr of the local instance -> SymmTensor
_COUNTER: Optional[torch.Tensor] = None
_UNIQUEID_BYTES = 128
_SIGNAL_SET, _CMP_GE = 0, 4


def SIGNAL_SET() -> int:
    return _SIGNAL_SET


def CMP_GE() -> int:
    return _CMP_GE


def nvshmem_uniqueid_size() -> int:
    return _UNIQUEID_BYTES


def nvshmem_get_uniqueid() -> bytes:
    return bytes(_UNIQUEID_BYTES)


def nvshmem_is_initialized() -> bool:
    return _HEAP is not None


def _heap():
    if _HEAP is None:
        raise RuntimeError("the one-sided transport is not initialised: call nvshmem_init() first")
    return _HEAP


def nvshmem_init() -> None:
    """Map the world group's symmetric heap (collective: every rank calls it)."""
    global _HEAP, _COUNTER
    if _HEAP is not None:
        return
    if not torch.cuda.is_available():
        raise RuntimeError("the one-sided transport needs a CUDA device")
    from .symm import SymmetricHeap
    nbytes = int(os.environ.get("FLUIDMOE_SHMEM_HEAP_BYTES", 1 << 30))
    _HEAP = SymmetricHeap(None, nbytes, torch.device("cuda", torch.cuda.current_device()))
    _COUNTER = torch.zeros(1, dtype=torch.int32, device=_HEAP.device)
    _HEAP.sync_group()


def nvshmem_init_with_uniqueid(my_pe: int, n_pes: int, uniqueid_bytes: bytes) -> None:
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    if (int(my_pe), int(n_pes)) != (rank, world):
        raise ValueError(f"PE {my_pe} of {n_pes} does not match rank {rank} of {world} of the process group")
    if len(uniqueid_bytes) != _UNIQUEID_BYTES:
        raise ValueError(f"unique id has {len(uniqueid_bytes)} bytes, expected {_UNIQUEID_BYTES}")
    nvshmem_init()


def nvshmem_finalize() -> None:
    global _HEAP, _COUNTER
    if _HEAP is not None:
        _HEAP.close()
    _HEAP, _COUNTER = None, None
    _ALLOCS.clear()


def nvshmem_my_pe() -> int:
    return _heap().rank


def nvshmem_n_pes() -> int:
    return _heap().world


def nvshmem_malloc_tensor(numel: int, dtype: torch.dtype) -> torch.Tensor:
    """A 1-D tensor at the same heap offset on every PE (collective; not zero-filled, like the
    reference's, fluid/csrc/nvshmem_ops.cpp:132-141)."""
    if int(numel) <= 0:
        raise ValueError("numel must be > 0")
    st = _heap().alloc((int(numel),), dtype, zero=False)
    _ALLOCS[st.local.data_ptr()] = st
    return st.local


def nvshmem_free_tensor(t: torch.Tensor) -> None:
    _heap()
    _ALLOCS.pop(t.data_ptr(), None)


def _locate(addr: int):
    for base, st in _ALLOCS.items():
        size = st.local.numel() * st.local.element_size()
        if base <= addr < base + size:
            return st, addr - base
    return None, 0


def nvshmem_ptr(t: torch.Tensor, pe: int) -> int:
    """Address of ``t`` (a heap tensor or a view into one) in PE ``pe``'s memory; 0 when ``t`` is
    not in the heap, as NVSHMEM answers for an unreachable address."""
    _heap()
    st, off = _locate(t.data_ptr())
    return 0 if st is None else int(st.peer_addrs[int(pe)]) + off


def putmem_signal_on_stream(dest_ptr: int, src: torch.Tensor, nbytes: int, sig_addr: int, sig_val: int,
                            sig_op: int, pe: int, stream_ptr: int) -> None:
    """Copy ``nbytes`` of ``src`` to ``dest_ptr`` and then store ``sig_val`` at ``sig_addr`` (both
    addresses in PE ``pe``'s memory, from ``nvshmem_ptr``), ordered on the stream.  The copy
    kernel's CTAs meet at one device counter of this module, so puts must not overlap in time:
    issue them on one stream, as the pairwise back-end does."""
    _heap()      # the peer is addressed through the two pointers; ``pe`` is kept for the signature
    if not dest_ptr or not sig_addr:
        raise ValueError("destination and signal addresses must not be null")
    if int(sig_op) != _SIGNAL_SET:
        raise NotImplementedError("only SIGNAL_SET is offered")
    if int(nbytes) % 16 != 0 or src.data_ptr() % 16 != 0 or int(dest_ptr) % 16 != 0:
        raise ValueError("payload and both buffers must be multiples of 16 bytes")
    if not 0 <= int(sig_val) < 1 << 31:
        raise ValueError("signal values are 32-bit here")
    from .. import _native
    _native.lib().put_signal(src.data_ptr(), int(nbytes), int(dest_ptr), int(sig_addr), int(sig_val), 16,
                             _COUNTER.data_ptr(), int(stream_ptr))


def signal_wait_until_on_stream(sig_addr: int, cmp_op: int, cmp_val: int, stream_ptr: int,
                                timeout_ms: float = 4000.0) -> None:
    """Stall the stream until the local signal word is >= ``cmp_val`` (bounded: after
    ``timeout_ms`` the kernel reports through the status word that ``check_status`` reads)."""
    heap = _heap()
    if not sig_addr:
        raise ValueError("signal address must not be null")
    if int(cmp_op) != _CMP_GE:
        raise NotImplementedError("only CMP_GE is offered")
    from .. import _native
    from ..ops.gemm import status_buffer
    _native.lib().wait_flag(int(sig_addr), int(cmp_val), int(timeout_ms * 1e6),
                            status_buffer(heap.device).data_ptr(), int(stream_ptr))


def quiet_on_stream(stream_ptr: int) -> None:
    _heap()
