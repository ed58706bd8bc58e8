"""Symmetric heap over NVLink peer memory.

Every rank allocates one block of the same size; every rank maps all the others' blocks. A
tensor allocated from the heap has the same byte offset on every rank, so a kernel can address
"this buffer on rank r" as ``peer_base(r) + offset``. Replaces the NVSHMEM symmetric heap of the
reference (maco/csrc/nvshmem_ops.cu:37-147, maco/comm/nvshmem_backend.py:54-104); handles are
exchanged through the process group's host-side (gloo) group instead of MPI.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from .. import _native as N

_current: Optional["SymmetricHeap"] = None
_ALIGN = 1024


class RangeAllocator:
    """Offsets inside a fixed range: first fit over a sorted, coalesced free list, bump allocation behind it.
    Deterministic, so ranks that issue the same calls get the same offsets. Pure Python (CPU-testable)."""

    def __init__(self, nbytes: int, align: int = _ALIGN):
        self.nbytes, self.align = int(nbytes), int(align)
        self.cursor = 0
        self.holes: List[tuple] = []        # sorted (start, size)
        self.live = {}                      # start -> size

    def alloc(self, nbytes: int) -> int:
        need = max(self.align, (int(nbytes) + self.align - 1) // self.align * self.align)
        for i, (fs, fsz) in enumerate(self.holes):
            if fsz >= need:
                if fsz == need:
                    self.holes.pop(i)
                else:
                    self.holes[i] = (fs + need, fsz - need)
                self.live[fs] = need
                return fs
        start = self.cursor
        if start + need > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} bytes at {start}, heap has {self.nbytes}. "
                              "Raise maco_b200.config.comm_buffer_size")
        self.cursor = start + need
        self.live[start] = need
        return start

    def free(self, start: int) -> tuple:
        size = self.live.pop(start, None)
        if size is None:
            raise ValueError("free(): not the start of a live allocation")
        holes = sorted(self.holes + [(start, size)])
        merged: List[tuple] = []
        for fs, fsz in holes:
            if merged and merged[-1][0] + merged[-1][1] == fs:
                merged[-1] = (merged[-1][0], merged[-1][1] + fsz)
            else:
                merged.append((fs, fsz))
        if merged and merged[-1][0] + merged[-1][1] == self.cursor:       # the top hole rejoins the bump region
            self.cursor = merged.pop()[0]
        self.holes = merged
        return start, size

    @property
    def free_bytes(self) -> int:
        return self.nbytes - self.cursor + sum(sz for _, sz in self.holes)


class _Span:
    """Exposes a raw device range through the CUDA array interface so torch can view it."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}
        self._owner = owner


class SymmetricHeap:
    def __init__(self, nbytes: int, rank: int, world: int, device: torch.device, exchange):
        """``exchange(obj) -> list`` gathers one Python object from every rank (rank order)."""
        lib = N.lib()
        P, U64 = ctypes.c_void_p, ctypes.c_ulonglong
        lib.maco_heap_create.restype = ctypes.c_int
        lib.maco_heap_create.argtypes = [U64, ctypes.POINTER(P), ctypes.c_char_p]
        lib.maco_heap_open.restype = ctypes.c_int
        lib.maco_heap_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(P)]
        lib.maco_heap_close.restype = ctypes.c_int
        lib.maco_heap_close.argtypes = [P]
        lib.maco_heap_destroy.restype = ctypes.c_int
        lib.maco_heap_destroy.argtypes = [P]
        self._lib = lib
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.nbytes = (int(nbytes) + _ALIGN - 1) // _ALIGN * _ALIGN
        torch.cuda.set_device(self.device)
        base = P()
        handle = ctypes.create_string_buffer(64)
        N.check(lib.maco_heap_create(self.nbytes, ctypes.byref(base), handle), "maco_heap_create")
        self._base = base.value
        handles = exchange(handle.raw)
        self._peer: List[int] = []
        for r, h in enumerate(handles):
            if r == rank:
                self._peer.append(self._base)
            else:
                pb = P()
                N.check(lib.maco_heap_open(h, ctypes.byref(pb)), f"maco_heap_open(rank {r})")
                self._peer.append(pb.value)
        self._ranges = RangeAllocator(self.nbytes)
        self._whole = torch.as_tensor(_Span(self._base, self.nbytes, self), device=self.device)
        self._closed = False
        exchange(b"ready")          # nobody touches a peer's heap before every rank has mapped it

    # ------------------------------------------------------------------ allocation
    def alloc(self, shape, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """First fit in the free list, else bump allocation. Every rank must run the same sequence of
        ``alloc`` / ``free`` calls with the same sizes, so a buffer has the same offset everywhere."""
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        start = self._ranges.alloc(nbytes)
        t = self._whole[start:start + nbytes].view(dtype).view(shape)
        if zero:
            t.zero_()
        return t

    def free(self, t: torch.Tensor) -> None:
        """Returns a buffer obtained from ``alloc`` to the heap and ZEROES it (event counters allocated later
        from this range must start at zero). Collective in effect: every rank frees the same buffers in the
        same order, after a device synchronisation and a host barrier (no kernel on any rank may still touch
        the range); the callers in ``parallel.collectives`` do both."""
        start, size = self._ranges.free(self.offset_of(t))
        self._whole[start:start + size].zero_()

    @property
    def free_bytes(self) -> int:
        return self._ranges.free_bytes

    # ------------------------------------------------------------------ addressing
    def owns(self, t: torch.Tensor) -> bool:
        if not isinstance(t, torch.Tensor) or not t.is_cuda or t.numel() == 0:
            return False
        p = t.data_ptr()
        return self._base <= p and p + t.numel() * t.element_size() <= self._base + self.nbytes

    def offset_of(self, t: torch.Tensor) -> int:
        if not self.owns(t):
            raise ValueError("tensor is not inside the symmetric heap")
        return t.data_ptr() - self._base

    def peer_base(self, r: int) -> int:
        return self._peer[r]

    def multicast_base(self) -> int:
        """Multicast (NVLS) address of the heap; 0 = not bound (plain peer loads/stores are used)."""
        return 0

    def peer_view(self, t: torch.Tensor, r: int) -> torch.Tensor:
        """The tensor at the same offset in rank ``r``'s heap (for tests and debugging)."""
        off = self.offset_of(t)
        nbytes = t.numel() * t.element_size()
        span = torch.as_tensor(_Span(self._peer[r] + off, nbytes, self), device=self.device)
        return span.view(t.dtype).view(t.shape)

    def close(self) -> None:
        if self._closed:
            return
        torch.cuda.synchronize(self.device)
        for r, p in enumerate(self._peer):
            if r != self.rank:
                self._lib.maco_heap_close(p)
        self._whole = None
        self._lib.maco_heap_destroy(self._base)
        self._closed = True


class LocalHeap:
    """A one-rank stand-in with the interface of :class:`SymmetricHeap`: programs whose tasks address
    buffers as "heap base + offset" (the MoE and fused-collective tasks) run unchanged on a single GPU."""

    def __init__(self, nbytes: int, device: Optional[torch.device] = None):
        self.rank, self.world = 0, 1
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + _ALIGN - 1) // _ALIGN * _ALIGN
        self._whole = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
        self._base = self._whole.data_ptr()
        self._ranges = RangeAllocator(self.nbytes)

    alloc = SymmetricHeap.alloc
    free = SymmetricHeap.free
    free_bytes = SymmetricHeap.free_bytes
    owns = SymmetricHeap.owns
    offset_of = SymmetricHeap.offset_of

    def peer_base(self, r: int) -> int:
        return self._base

    def multicast_base(self) -> int:
        return 0

    def peer_view(self, t: torch.Tensor, r: int) -> torch.Tensor:
        return t

    def close(self) -> None:
        self._whole = None


def init_heap(nbytes: Optional[int] = None) -> SymmetricHeap:
    """Creates the process-wide heap over the current process group (idempotent)."""
    global _current
    if _current is not None:
        return _current
    from ..comm.process_group import ProcessGroupManager
    from ..config import config
    pgm = ProcessGroupManager()
    if not pgm.is_initialized:
        pgm.init_process_group()
    if pgm.device.type != "cuda":
        raise RuntimeError("the symmetric heap needs CUDA devices")
    _current = SymmetricHeap(nbytes or config.comm_buffer_bytes, pgm.rank, pgm.world_size, pgm.device,
                             pgm.all_gather_object)
    return _current


def current_heap() -> Optional[SymmetricHeap]:
    return _current


def destroy_heap(collective: bool = True) -> None:
    """Unmaps the peers and frees the heap. ``collective=False`` skips the barrier (use it after a peer
    was lost: a barrier with a dead rank would never return)."""
    global _current
    if _current is not None:
        from ..comm.process_group import barrier
        try:
            if collective:
                barrier()
        except Exception:
            pass
        from . import collectives
        collectives.clear_cache()
        _current.close()
        _current = None
