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


def _exchange_fds(serve_fd: Optional[int], fetch_from: List[int], rank: int, world: int, exchange, tag: str) -> dict:
    """Passes file descriptors between the ranks of one node over Unix-domain sockets (SCM_RIGHTS): every rank
    that has a descriptor serves it to whoever connects, and fetches one from each rank in ``fetch_from``.
    ``exchange`` publishes the socket names. Returns {source rank: received descriptor}."""
    import os
    import socket
    import threading
    name = f"\0maco_b200_{tag}_{os.getpid()}_{rank}"           # abstract namespace: nothing to unlink
    server = None
    n_clients = 0
    if serve_fd is not None:
        server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        server.bind(name)
        server.listen(world)
    names = exchange((name if serve_fd is not None else None, list(fetch_from)))
    if serve_fd is not None:
        n_clients = sum(1 for r, (_, wants) in enumerate(names) if r != rank and rank in wants)

    def serve():
        for _ in range(n_clients):
            conn, _ = server.accept()
            with conn:
                conn.recv(4)
                socket.send_fds(conn, [b"fd"], [serve_fd])

    th = None
    if server is not None and n_clients:
        th = threading.Thread(target=serve, daemon=True)
        th.start()
    got = {}
    for src in fetch_from:
        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
            c.settimeout(60.0)
            c.connect(names[src][0])
            c.sendall(rank.to_bytes(4, "little"))
            _, fds, _, _ = socket.recv_fds(c, 16, 1)
            got[src] = fds[0]
    if th is not None:
        th.join(60.0)
    if server is not None:
        server.close()
    return got


class SymmetricHeap:
    def __init__(self, nbytes: int, rank: int, world: int, device: torch.device, exchange, mode: Optional[str] = None):
        """``exchange(obj) -> list`` gathers one Python object from every rank (rank order).

        ``mode``: "ipc" = cudaMalloc + CUDA IPC (plain peer loads / stores only); "vmm" = CUDA virtual-memory
        allocations shared through file descriptors; "nvls" = "vmm" plus one NVSwitch multicast object over
        all ranks' heaps (``multicast_base()`` is then non-zero and kernels may use multimem instructions);
        None = the environment variable MACO_HEAP if set, else "nvls" where the devices support it (and
        MACO_NVLS is not 0), falling back to "vmm" and then "ipc". All ranks take the same decision."""
        import os
        lib = N.lib()
        P, U64, I = ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_int
        lib.maco_heap_create.restype = ctypes.c_int
        lib.maco_heap_create.argtypes = [U64, ctypes.POINTER(P), ctypes.c_char_p]
        lib.maco_heap_open.restype = ctypes.c_int
        lib.maco_heap_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(P)]
        lib.maco_heap_close.restype = ctypes.c_int
        lib.maco_heap_close.argtypes = [P]
        lib.maco_heap_destroy.restype = ctypes.c_int
        lib.maco_heap_destroy.argtypes = [P]
        lib.maco_vheap_supported.argtypes = [ctypes.POINTER(I)]
        lib.maco_vheap_create.argtypes = [ctypes.POINTER(U64), I, I, I, ctypes.POINTER(P), ctypes.POINTER(I)]
        lib.maco_vheap_import.argtypes = [I, I, ctypes.POINTER(P)]
        lib.maco_vheap_mc_create.argtypes = [ctypes.POINTER(I)]
        lib.maco_vheap_mc_import.argtypes = [I]
        lib.maco_vheap_mc_map.argtypes = [ctypes.POINTER(P)]
        self._lib = lib
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.nbytes = (int(nbytes) + _ALIGN - 1) // _ALIGN * _ALIGN
        torch.cuda.set_device(self.device)
        self._mc_base = 0
        mode = mode or os.environ.get("MACO_HEAP") or None
        if mode == "auto":
            mode = None
        mc_flag = I(0)
        fd_ok = bool(lib.maco_vheap_supported(ctypes.byref(mc_flag)))
        nvls_ok = bool(mc_flag.value) and os.environ.get("MACO_NVLS", "1") != "0" and world > 1
        if mode is None:
            mode = "nvls" if (fd_ok and nvls_ok) else ("vmm" if fd_ok else "ipc")
        if mode not in ("ipc", "vmm", "nvls"):
            raise ValueError(f"unknown heap mode {mode!r}")
        if mode != "ipc" and not fd_ok:
            mode = "ipc"
        if mode == "nvls" and not nvls_ok:
            mode = "vmm"
        # the ranks agree on the weakest mode any of them can offer
        order = {"ipc": 0, "vmm": 1, "nvls": 2}
        mode = min(exchange(mode), key=order.get)
        self.mode = mode
        if mode == "ipc":
            self._init_ipc(exchange)
        else:
            self._init_vmm(exchange, want_multicast=(mode == "nvls"))
        self._ranges = RangeAllocator(self.nbytes)
        self._whole = torch.as_tensor(_Span(self._base, self.nbytes, self), device=self.device)
        self._closed = False
        exchange(b"ready")          # nobody touches a peer's heap before every rank has mapped it

    def _init_ipc(self, exchange) -> None:
        lib, P = self._lib, ctypes.c_void_p
        base = P()
        handle = ctypes.create_string_buffer(64)
        N.check(lib.maco_heap_create(self.nbytes, ctypes.byref(base), handle), "maco_heap_create")
        self._base = base.value
        handles = exchange(handle.raw)
        self._peer: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self._peer.append(self._base)
            else:
                pb = P()
                N.check(lib.maco_heap_open(h, ctypes.byref(pb)), f"maco_heap_open(rank {r})")
                self._peer.append(pb.value)

    def _init_vmm(self, exchange, want_multicast: bool) -> None:
        import os
        lib, P, I = self._lib, ctypes.c_void_p, ctypes.c_int
        size = ctypes.c_ulonglong(self.nbytes)
        base, fd = P(), I(-1)
        N.check(lib.maco_vheap_create(ctypes.byref(size), self.rank, self.world, int(want_multicast), ctypes.byref(base),
                                      ctypes.byref(fd)), "maco_vheap_create")
        self.nbytes = int(size.value)
        self._base = base.value
        others = [r for r in range(self.world) if r != self.rank]
        got = _exchange_fds(fd.value, others, self.rank, self.world, exchange, "heap")
        self._peer = [0] * self.world
        self._peer[self.rank] = self._base
        for r in others:
            pb = P()
            N.check(lib.maco_vheap_import(r, got[r], ctypes.byref(pb)), f"maco_vheap_import(rank {r})")
            self._peer[r] = pb.value
            os.close(got[r])
        exchange(b"imported")
        os.close(fd.value)
        if not want_multicast:
            return
        # multicast object: created by rank 0, joined by every device, then every rank binds its own allocation.
        # A step that fails anywhere leaves the whole job on plain peer access (the ranks vote after each step).
        def all_ok(rc: int) -> bool:
            return all(v == 0 for v in exchange(int(rc)))
        mc_fd = I(-1)
        rc = lib.maco_vheap_mc_create(ctypes.byref(mc_fd)) if self.rank == 0 else 0
        if not all_ok(rc):
            return
        got = _exchange_fds(mc_fd.value if self.rank == 0 else None, [0] if self.rank != 0 else [], self.rank, self.world,
                            exchange, "mc")
        rc = 0
        if self.rank != 0:
            rc = lib.maco_vheap_mc_import(got[0])
            os.close(got[0])
        ok = all_ok(rc)
        if self.rank == 0:
            os.close(mc_fd.value)
        if not ok or not all_ok(lib.maco_vheap_mc_add_device()):
            return
        if not all_ok(lib.maco_vheap_mc_bind()):
            return
        mc = P()
        if not all_ok(lib.maco_vheap_mc_map(ctypes.byref(mc))):
            return
        self._mc_base = mc.value

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
        return self._mc_base

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
        self._whole = None
        if self.mode == "ipc":
            for r, p in enumerate(self._peer):
                if r != self.rank:
                    self._lib.maco_heap_close(p)
            self._lib.maco_heap_destroy(self._base)
        else:
            self._lib.maco_vheap_destroy()
        self._mc_base = 0
        self._closed = True


class PlanningHeap:
    """Host-memory stand-in for one rank of a ``world``-rank symmetric heap, for planning without GPUs: model
    builders on a CPU device take it as their ``heap``, allocate their buffers from it (the same offsets on every
    rank, as the real heap guarantees) and produce the task lists that ``ops.megakernel.simulate_static_queues`` and
    ``estimate_makespan`` run. Nothing is ever copied between ranks; the memory is untouched virtual address space."""

    def __init__(self, rank: int, world: int, nbytes: int = 1 << 30):
        self.rank, self.world = int(rank), int(world)
        self.device = torch.device("cpu")
        self.mode = "planning"
        self.nbytes = (int(nbytes) + _ALIGN - 1) // _ALIGN * _ALIGN
        self._whole = torch.empty(self.nbytes, dtype=torch.uint8)
        self._base = self._whole.data_ptr()
        self._ranges = RangeAllocator(self.nbytes)

    def alloc(self, shape, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        return SymmetricHeap.alloc(self, shape, dtype, False)        # never touch the pages: planning only

    def free(self, t: torch.Tensor) -> None:
        self._ranges.free(self.offset_of(t))

    free_bytes = SymmetricHeap.free_bytes
    offset_of = SymmetricHeap.offset_of

    def owns(self, t: torch.Tensor) -> bool:
        if not isinstance(t, torch.Tensor) or t.numel() == 0:
            return False
        p = t.data_ptr()
        return self._base <= p and p + t.numel() * t.element_size() <= self._base + self.nbytes

    def peer_base(self, r: int) -> int:
        return self._base

    def multicast_base(self) -> int:
        return 0


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
                             pgm.all_gather_object, mode=None if config.heap_mode == "auto" else config.heap_mode)
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
