"""Symmetric device memory: one buffer per rank, every rank's buffer mapped on every rank.

The buffers back the flat gradient / parameter stores and the signal pads of the fused
multi-GPU kernels.  Allocation and CUDA-IPC mapping are done by the native library
(``csrc/symm.cpp``); this module moves the 64-byte handles through the process group
(a host-side, one-time exchange) and keeps the mappings alive.
"""

from __future__ import annotations

import os
from typing import List, Optional

import torch

from .. import _native

SIGNAL_WORDS = 18          # 8 entry flags, 8 exit flags, go word, done counter
MAX_PEERS = 8
GUARD_BYTES = 256          # canary words before and after the payload when APEXW_B200_DEBUG=1
_CANARY = 0x5A


def _dist_ready(group=None) -> bool:
    import torch.distributed as dist
    return dist.is_available() and dist.is_initialized()


class SymmetricBuffer:
    """``nbytes`` of zero-filled device memory on this rank plus mappings of every peer's copy.

    Construction is collective over ``group`` when ``torch.distributed`` is initialised with
    more than one rank; with one rank it is a plain allocation.

    The memory belongs to a reference-counted native object.  Every tensor from :meth:`tensor` (and every
    view of it, such as model parameters re-pointed into a flat buffer) holds a reference through its
    storage, so the memory outlives this Python object for as long as anything still reads or writes it;
    it is released, peer mappings first, when the last holder goes.
    """

    def __init__(self, nbytes: int, device: torch.device, group=None):
        self._nat = _native.require()
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        self._dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        # debug build of the buffer: guard bands around the payload, filled with a pattern that no kernel writes;
        # check_canaries() tells whether a peer kernel stored outside the payload
        self._guard = GUARD_BYTES if os.environ.get("APEXW_B200_DEBUG", "0") not in ("", "0") else 0
        self._alloc = self._nat.SymmAlloc(self.nbytes + 2 * self._guard, self._dev_index)
        self._base_ptr = self._alloc.ptr
        self.local_ptr = self._base_ptr + self._guard
        if self._guard:
            for off in (0, self._guard + self.nbytes):
                self._nat.symm_tensor(self._alloc, self._base_ptr + off, [self._guard], torch.uint8).fill_(_CANARY)
        self.rank, self.world = 0, 1
        self.peer_ptrs: List[int] = [self.local_ptr]
        if _dist_ready():
            import torch.distributed as dist
            world = dist.get_world_size(group)
            if world > 1:
                if world > MAX_PEERS:
                    raise RuntimeError(f"symmetric buffers support at most {MAX_PEERS} ranks per group, got {world}")
                self.rank, self.world = dist.get_rank(group), world
                handles: List[Optional[bytes]] = [None] * world
                dist.all_gather_object(handles, bytes(self._alloc.handle), group=group)
                self.peer_ptrs = []
                for r, h in enumerate(handles):
                    if r == self.rank:
                        self.peer_ptrs.append(self.local_ptr)
                    else:
                        self.peer_ptrs.append(self._alloc.open_peer(h) + self._guard)   # every rank uses the same guard size
                dist.barrier(group=group)

    def tensor(self, dtype: torch.dtype, numel: int, byte_offset: int = 0, rank: Optional[int] = None) -> torch.Tensor:
        """A tensor view of this rank's buffer (or of ``rank``'s mapping).  Its storage keeps the allocation alive."""
        itemsize = torch.empty((), dtype=dtype).element_size()
        if byte_offset % itemsize or byte_offset + numel * itemsize > self.nbytes:
            raise ValueError("view exceeds the symmetric buffer")
        if self._alloc is None:
            raise RuntimeError("this SymmetricBuffer was closed")
        base = self.local_ptr if rank is None else self.peer_ptrs[rank]
        return self._nat.symm_tensor(self._alloc, base + byte_offset, [numel], dtype)

    def check_canaries(self) -> bool:
        """True when the guard bands of this rank's buffer still hold their pattern (always True without
        ``APEXW_B200_DEBUG=1``, which is what allocates them)."""
        if not self._guard or self._alloc is None:
            return True
        ok = True
        for off in (0, self._guard + self.nbytes):
            band = self._nat.symm_tensor(self._alloc, self._base_ptr + off, [self._guard], torch.uint8)
            ok = ok and bool((band == _CANARY).all().item())
        return ok

    def close(self) -> None:
        """Drop this object's reference.  The memory itself is released only when no tensor uses it any more."""
        self._alloc = None
        self.peer_ptrs = []


class MulticastBuffer:
    """Symmetric memory with an NVSwitch multicast address on top of the per-rank addresses.

    ``multicast_ptr`` names the same byte offset in EVERY rank's buffer at once: a ``multimem.ld_reduce`` on it
    returns the sum over ranks, reduced inside the switch, and a ``multimem.st`` writes all ranks' copies with one
    store (NVLS).  The per-rank ``peer_ptrs`` work as in :class:`SymmetricBuffer`.  Allocation, handle exchange and
    the multicast binding are ``torch.distributed._symmetric_memory``'s (host-side plumbing); the kernels that use
    the addresses are this library's.  Construction is collective over ``group``.  ``supported`` is False - and the
    object unusable - where the platform gives no multicast address; callers then stay on plain peer loads.

    Every rank of the group has to leave the job together: a rank that dies while its memory is bound to the
    multicast object can raise NVLink faults on its peers, so failure tests never run on this kind of buffer.
    """

    def __init__(self, nbytes: int, device: torch.device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        self.supported = False
        self.multicast_ptr = 0
        self.peer_ptrs: List[int] = []
        self.local_ptr = 0
        if not _dist_ready():
            return
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        try:
            self._base = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            handle = symm_mem.rendezvous(self._base, group)
            self._handle = handle
            self.peer_ptrs = [int(p) for p in handle.buffer_ptrs]
            self.multicast_ptr = int(handle.multicast_ptr)
            self.local_ptr = self.peer_ptrs[self.rank]
            self._base.zero_()
            self.supported = self.multicast_ptr != 0 and self.local_ptr == self._base.data_ptr()
        except Exception as exc:      # no fabric / multicast support: the caller falls back
            self._error = f"{type(exc).__name__}: {exc}"
            self.supported = False

    def tensor(self, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        """A tensor view of this rank's buffer; its storage is the allocation itself."""
        itemsize = torch.empty((), dtype=dtype).element_size()
        if byte_offset % itemsize or byte_offset + numel * itemsize > self.nbytes:
            raise ValueError("view exceeds the symmetric buffer")
        return self._base[byte_offset:byte_offset + numel * itemsize].view(dtype)

    def check_canaries(self) -> bool:
        return True


def live_allocations() -> int:
    """Number of symmetric allocations of this process that have not been released yet."""
    return int(_native.require().symm_live_allocations())
