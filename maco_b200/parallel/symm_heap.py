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
        self._cursor = 0
        self._whole = torch.as_tensor(_Span(self._base, self.nbytes, self), device=self.device)
        self._closed = False
        exchange(b"ready")          # nobody touches a peer's heap before every rank has mapped it

    # ------------------------------------------------------------------ allocation
    def alloc(self, shape, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """Bump allocation; every rank must allocate the same sequence of sizes."""
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        start = (self._cursor + _ALIGN - 1) // _ALIGN * _ALIGN
        if start + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} bytes at {start}, heap has {self.nbytes}. "
                              "Raise maco_b200.config.comm_buffer_size")
        self._cursor = start + nbytes
        t = self._whole[start:start + nbytes].view(dtype).view(shape)
        if zero:
            t.zero_()
        return t

    def mark(self) -> int:
        return self._cursor

    def release_to(self, mark: int) -> None:
        """Frees everything allocated after ``mark`` (stack discipline, same on every rank)."""
        self._cursor = mark

    @property
    def free_bytes(self) -> int:
        return self.nbytes - self._cursor

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
        self._cursor = 0

    alloc = SymmetricHeap.alloc
    owns = SymmetricHeap.owns
    offset_of = SymmetricHeap.offset_of
    mark = SymmetricHeap.mark
    release_to = SymmetricHeap.release_to

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
