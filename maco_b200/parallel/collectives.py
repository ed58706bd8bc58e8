"""Stand-alone collectives served by the persistent kernel's communication tasks.

Each call builds (once, then caches) a small program over buffers of the symmetric heap and launches
it: all ranks' kernels push (or pull) over NVLink peer memory and synchronise through event counters
in the heap. These back ``comm.patterns`` when ``config.backend == "peer"``, and the ``nvshmem_*``
compatibility calls. NCCL stays available as the baseline (``comm.nccl_ops``).

Ordering against the caller's other work. A program that writes into a peer's buffer opens with a
handshake: every rank's kernel first bumps a ``ready`` counter on all ranks, and no data task starts
before the counter shows that EVERY rank's kernel of this call is running. A kernel starts only after
everything queued before it on its stream, so when a peer's data arrives, whatever the receiving rank
did with the buffer's previous contents (a copy of the last result, an attention kernel) has finished.
That holds across different programs sharing a buffer too, because all ranks issue collectives in
the same order. Programs in which peers READ this rank's memory (reduce-scatter) also close with a
barrier: the kernel does not end before every rank has finished reading, so the caller may overwrite
its input as soon as the call's kernel is done.

The cache is bounded (``MAX_CACHED_PROGRAMS``, least recently used first out). Evicting a program is
collective by construction (all ranks run the same call sequence, hence the same eviction): device
synchronise, host barrier, free and zero the program's heap buffers.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _native as N
from ..ops.megakernel import COMM_ALLREDUCE_MC, COMM_PUSH, COMM_REDUCE_PULL, Program, ProgramBuilder, _pack_comm
from ..task_graph.nodes import TaskType
from . import fused
from .symm_heap import current_heap

MAX_CACHED_PROGRAMS = 64

Wait = Tuple[int, int, bool, bool]


class _Entry:
    """A cached program with the heap buffers that belong to it alone."""

    def __init__(self, programs: List[Program], buffers: List[torch.Tensor]):
        self.programs, self.buffers, self.calls = programs, buffers, 0


_cache: "OrderedDict[tuple, _Entry]" = OrderedDict()


def _heap():
    h = current_heap()
    if h is None:
        raise RuntimeError("the symmetric heap is not initialised; call maco_b200.init_nvshmem() / init()")
    return h


def _builder(heap, workers: int = 16) -> ProgramBuilder:
    return ProgramBuilder(heap.device, num_workers=workers, mode="static", heap=heap)


def _open(b: ProgramBuilder) -> Wait:
    """Opening handshake: returns the condition "every rank's kernel of this launch is running"."""
    ready = b.new_event()
    b.add_task(int(TaskType.PEER_BARRIER), b"", signal_peer=-2, signal_peer_event=ready)
    return (ready, b.heap.world, True, False)


def _close(b: ProgramBuilder, waits: Sequence[Wait]) -> None:
    """Closing barrier: when ``waits`` hold locally, tell every rank; the kernel ends only when every rank said so."""
    closed = b.new_event()
    b.add_task(int(TaskType.PEER_BARRIER), b"", waits=b.join(list(waits)), signal_peer=-2, signal_peer_event=closed)
    b.add_task(int(TaskType.NOP), b"", waits=[(closed, b.heap.world, True, False)])


def _wait_local(b: ProgramBuilder, waits: Sequence[Wait]) -> None:
    """Last task of a push program: the kernel ends once everything this rank expects has arrived."""
    if waits:
        b.add_task(int(TaskType.NOP), b"", waits=b.join(list(waits)))


def _evict_one() -> None:
    heap = _heap()
    _, entry = _cache.popitem(last=False)
    torch.cuda.synchronize(heap.device)
    from ..comm.process_group import barrier
    barrier()                               # no rank's kernel still touches the buffers
    for p in entry.programs:
        p.free_heap()
    for buf in entry.buffers:
        heap.free(buf)
    barrier()                               # nobody reuses the range before every rank has zeroed it


def _lookup(key: tuple) -> Optional[_Entry]:
    e = _cache.get(key)
    if e is not None:
        _cache.move_to_end(key)
    return e


def _store(key: tuple, entry: _Entry) -> _Entry:
    while len(_cache) >= MAX_CACHED_PROGRAMS:
        _evict_one()
    _cache[key] = entry
    return entry


def all_reduce(t: torch.Tensor, avg: bool = False, multicast: Optional[bool] = None) -> torch.Tensor:
    """In-place sum (or mean) of heap tensor ``t`` over all ranks.

    With a multicast-bound heap (``multicast`` None = use it when there is one): chunk c belongs to rank
    c % world, which loads the sum of every rank's copy with multimem.ld_reduce (the switch adds, in fp32
    for 16-bit types) and stores the result to every copy with multimem.st: each byte crosses this GPU's
    links about once in each direction. The kernels open with the handshake (every rank's buffer is ready)
    and a rank's kernel ends when all chunks of its copy are final, which is also when nobody reads it any more.

    Without: every rank stores its copy of a chunk into the owner's staging slot, the owner sums the slots in
    fp32 and stores the result into ``t`` on every rank (no remote reads). The owner's stores can only start
    after every rank's kernel has contributed, so they never hit a buffer whose owner is still preparing it."""
    heap = _heap()
    if multicast is None:
        multicast = bool(heap.multicast_base())
    key = ("ar", heap.offset_of(t), t.numel(), t.dtype, avg, multicast)
    e = _lookup(key)
    if e is None and multicast:
        nbytes = t.numel() * t.element_size()
        if nbytes % 16:
            raise ValueError("all-reduce buffers must be a multiple of 16 bytes")
        chunk = 128 << 10
        n_chunks = -(-nbytes // chunk)
        # nothing else runs beside a stand-alone collective: one chunk per worker, every SM if there are enough chunks
        b = _builder(heap, workers=max(1, min(N.lib().maco_sm_count(), -(-n_chunks // heap.world))))
        ready = _open(b)
        done = b.new_event()
        off = heap.offset_of(t)
        for c in range(n_chunks):
            if c % heap.world != heap.rank:
                continue
            c0 = c * chunk
            row, rows = _push_rows(min(chunk, nbytes - c0))
            raw = _pack_comm(off + c0, off + c0, row, row, row, rows, N.DTYPE_CODE[t.dtype], -1, COMM_ALLREDUCE_MC,
                             scale=(1.0 / heap.world if avg else 1.0))
            b.add_task(int(TaskType.ALLREDUCE), raw, waits=[ready], signal_peer=-4, signal_peer_event=done)
        _wait_local(b, [(done, n_chunks, True, False)])
        e = _store(key, _Entry([b.build()], []))
    if e is None:
        nbytes = t.numel() * t.element_size()
        chunk = 256 << 10
        n_chunks = -(-nbytes // chunk)
        per_owner = -(-n_chunks // heap.world)
        # staging of its own per program: a faster rank's next call (another program) may already be storing
        # into the owner's slots while the owner still sums this call's
        staging = heap.alloc((heap.world * per_owner * chunk,), torch.uint8)
        b = _builder(heap, workers=max(1, min(N.lib().maco_sm_count(), 2 * n_chunks)))
        fence = fused.epoch_fence_event(b)
        done, n = fused.allreduce_push_tasks(b, t.view(-1), staging, avg=avg, chunk_bytes=chunk, fence=fence)
        fused.epoch_fence_signal(b, [(done, n, True, False)])
        e = _store(key, _Entry([b.build()], [staging]))
    e.programs[0].run()
    return t


_staging: Dict[tuple, torch.Tensor] = {}


def _staging_like(t: torch.Tensor, tag: str, shape=None) -> torch.Tensor:
    """Heap buffer for tensors that live outside the heap, one per (tag, shape, dtype), reused by later calls."""
    heap = _heap()
    shape = tuple(shape if shape is not None else t.shape)
    key = (tag, shape, t.dtype)
    buf = _staging.get(key)
    if buf is None:
        buf = _staging[key] = heap.alloc(shape, t.dtype)
    return buf


def all_reduce_any(t: torch.Tensor, avg: bool = False) -> torch.Tensor:
    """All-reduce of any CUDA tensor: staged through a heap buffer when ``t`` lives outside the heap."""
    heap = _heap()
    if heap.owns(t) and t.is_contiguous():
        return all_reduce(t, avg)
    if t.dtype not in N.DTYPE_CODE:
        raise ValueError(f"unsupported dtype {t.dtype}")
    numel = (t.numel() * t.element_size() + 15) // 16 * 16 // t.element_size()
    buf = _staging_like(t, "ar", (numel,))
    if numel != t.numel():
        buf[t.numel():].zero_()
    buf[: t.numel()].copy_(t.reshape(-1))
    all_reduce(buf, avg)
    t.copy_(buf[: t.numel()].view(t.shape))
    return t


def device_barrier() -> None:
    """All ranks' kernels meet: each bumps every rank's counter and waits for ``world`` bumps."""
    heap = _heap()
    key = ("barrier",)
    e = _lookup(key)
    if e is None:
        b = _builder(heap, workers=1)
        ev = b.new_event()
        b.add_task(int(TaskType.PEER_BARRIER), b"", signal_peer=-2, signal_peer_event=ev)
        b.add_task(int(TaskType.NOP), b"", waits=[(ev, heap.world, True, False)])
        e = _store(key, _Entry([b.build()], []))
    e.programs[0].run()


def all_gather(shard: torch.Tensor, gathered: torch.Tensor) -> torch.Tensor:
    """``gathered`` [world*rows, cols] <- every rank's ``shard`` [rows, cols]; both in the heap."""
    heap = _heap()
    key = ("ag", heap.offset_of(shard), heap.offset_of(gathered), tuple(shard.shape), shard.dtype)
    e = _lookup(key)
    if e is None:
        b = _builder(heap)
        ev = fused.allgather_push(b, shard, gathered, fence=_open(b))
        _wait_local(b, [(ev_, c, True, False) for ev_, c in ev.row_events if c])
        e = _store(key, _Entry([b.build()], []))
    e.programs[0].run()
    return gathered


def _a2a4d_out_shape(t: torch.Tensor, P: int, scatter_dim: int, gather_dim: int) -> tuple:
    if (scatter_dim, gather_dim) == (2, 1):
        B, s, H, D = t.shape
        if H % P:
            raise ValueError(f"heads ({H}) not divisible by world size {P}")
        return (B, s * P, H // P, D)
    if (scatter_dim, gather_dim) == (1, 2):
        B, S, h, D = t.shape
        if S % P:
            raise ValueError(f"sequence ({S}) not divisible by world size {P}")
        return (B, S // P, h * P, D)
    raise ValueError("all_to_all_4d supports (scatter, gather) = (2, 1) or (1, 2)")


def _a2a4d_program(heap, t: torch.Tensor, out: torch.Tensor, scatter_dim: int, gather_dim: int) -> Program:
    P, r = heap.world, heap.rank
    b = _builder(heap)
    ready = _open(b)
    done = b.new_event()
    es = t.element_size()
    src, dst = heap.offset_of(t), heap.offset_of(out)
    n_tasks = 0
    for q in range(P):
        for bi in range(t.shape[0]):
            if (scatter_dim, gather_dim) == (2, 1):
                _, s, H, D = t.shape
                hp = H // P
                row_bytes = hp * D * es                      # the heads rank q keeps, for one position
                s_off = src + (bi * s * H * D + q * hp * D) * es
                d_off = dst + (bi * s * P * hp * D + r * s * hp * D) * es
                rows, s_stride, d_stride = s, H * D * es, hp * D * es
            else:
                _, S, h, D = t.shape
                sp = S // P
                row_bytes = h * D * es
                s_off = src + (bi * S * h * D + q * sp * h * D) * es
                d_off = dst + (bi * sp * P * h * D + r * h * D) * es
                rows, s_stride, d_stride = sp, h * D * es, P * h * D * es
            raw = _pack_comm(s_off, d_off, s_stride, d_stride, row_bytes, rows, N.DTYPE_CODE[t.dtype], q, COMM_PUSH)
            b.add_task(int(TaskType.ALL_TO_ALL), raw, waits=[ready], signal_peer=q, signal_peer_event=done)
            n_tasks += 1
    _wait_local(b, [(done, n_tasks, True, False)])
    return b.build()


def all_to_all_4d(t: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ulysses layout switch on a heap tensor, written straight into the destination layout:
    (2,1): [B, S/P, H, D] -> [B, S, H/P, D];  (1,2): [B, S, H/P, D] -> [B, S/P, H, D].
    Each (batch, sequence position, destination rank) slice is one row of a strided 2-D push, so
    there are no pack / unpack passes (the reference packs, exchanges and unpacks:
    maco/comm/patterns.py:400-436, maco/csrc/nvshmem_ops.cu:399-494).

    ``out`` is a heap tensor of the result shape. Without it the result lands in one of TWO buffers that
    belong to this input tensor alone and alternate between calls: the tensor returned by a call stays
    intact until the second-next call on the same input (q, k and v, being different inputs, never share
    a buffer)."""
    heap = _heap()
    out_shape = _a2a4d_out_shape(t, heap.world, scatter_dim, gather_dim)
    if out is not None:
        if tuple(out.shape) != out_shape or out.dtype != t.dtype or not heap.owns(out) or not out.is_contiguous():
            raise ValueError(f"all_to_all_4d: out must be a contiguous heap tensor of shape {out_shape} and dtype {t.dtype}")
        key = ("a2a", heap.offset_of(t), heap.offset_of(out), tuple(t.shape), t.dtype, scatter_dim, gather_dim)
        e = _lookup(key)
        if e is None:
            e = _store(key, _Entry([_a2a4d_program(heap, t, out, scatter_dim, gather_dim)], []))
        e.programs[0].run()
        return out
    key = ("a2a", heap.offset_of(t), -1, tuple(t.shape), t.dtype, scatter_dim, gather_dim)
    e = _lookup(key)
    if e is None:
        outs = [heap.alloc(out_shape, t.dtype) for _ in range(2)]
        e = _store(key, _Entry([_a2a4d_program(heap, t, o, scatter_dim, gather_dim) for o in outs], outs))
    i = e.calls & 1
    e.calls += 1
    e.programs[i].run()
    return e.buffers[i]


def all_to_all_4d_any(t: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1) -> torch.Tensor:
    """Ulysses layout switch of any CUDA tensor; returns a fresh tensor outside the heap."""
    heap = _heap()
    if not (heap.owns(t) and t.is_contiguous()):
        buf = _staging_like(t, "a2a_in")
        buf.copy_(t)
        t = buf
    out_shape = _a2a4d_out_shape(t, heap.world, scatter_dim, gather_dim)
    out = _staging_like(t, f"a2a_out{scatter_dim}{gather_dim}", out_shape)
    return all_to_all_4d(t, scatter_dim, gather_dim, out=out).clone()


def _chunks(nbytes: int, chunk: int = 1 << 20):
    """(offset, bytes) pieces of a contiguous byte range; every piece a multiple of 16 bytes."""
    off = 0
    while off < nbytes:
        n = min(chunk, nbytes - off)
        yield off, n
        off += n


def _push_rows(nbytes: int) -> Tuple[int, int]:
    """(row_bytes, rows) describing ``nbytes`` contiguous bytes as a 2-D block of whole 16-byte vectors."""
    row = 16384 if nbytes % 16384 == 0 else 16
    return row, nbytes // row


def broadcast(t: torch.Tensor, src: int = 0) -> torch.Tensor:
    """Heap tensor ``t`` of rank ``src`` is copied into ``t`` of every other rank (the source pushes
    1 MB pieces to all peers from inside the kernel; receivers wait on a counter)."""
    heap = _heap()
    nbytes = t.numel() * t.element_size()
    if nbytes % 16 or not t.is_contiguous():
        raise ValueError("broadcast needs a contiguous tensor of a multiple of 16 bytes")
    key = ("bc", heap.offset_of(t), nbytes, src)
    e = _lookup(key)
    if e is None:
        b = _builder(heap)
        ready = _open(b)
        done = b.new_event()
        off = heap.offset_of(t)
        pieces = list(_chunks(nbytes))
        if heap.rank == src:
            for o, n in pieces:
                row, rows = _push_rows(n)
                raw = _pack_comm(off + o, off + o, row, row, row, rows, N.DTYPE_CODE.get(t.dtype, 0), -1, COMM_PUSH)
                b.add_task(int(TaskType.BROADCAST), raw, waits=[ready], signal_peer=-2, signal_peer_event=done)
        _wait_local(b, [(done, len(pieces), True, False)])
        e = _store(key, _Entry([b.build()], []))
    e.programs[0].run()
    return t


def reduce_scatter(inp: torch.Tensor, out: torch.Tensor, avg: bool = False) -> torch.Tensor:
    """``out`` [rows, ...] <- sum over ranks of block ``rank`` of their ``inp`` [world*rows, ...]; both in
    the heap. Every rank pulls its block from all ranks over NVLink and sums in fp32; the kernels leave
    together, so ``inp`` may be overwritten as soon as the call's kernel has finished."""
    heap = _heap()
    P, r = heap.world, heap.rank
    nbytes = out.numel() * out.element_size()
    if inp.numel() != out.numel() * P or nbytes % 16 or inp.dtype != out.dtype:
        raise ValueError("reduce_scatter: inp must hold world blocks of out's size (a multiple of 16 bytes)")
    key = ("rs", heap.offset_of(inp), heap.offset_of(out), nbytes, out.dtype, avg)
    e = _lookup(key)
    if e is None:
        b = _builder(heap)
        ready = _open(b)
        done = b.new_event()
        src, dst = heap.offset_of(inp) + r * nbytes, heap.offset_of(out)
        n = 0
        for o, nb in _chunks(nbytes, 256 << 10):
            row, rows = _push_rows(nb)
            raw = _pack_comm(src + o, dst + o, row, row, row, rows, N.DTYPE_CODE[out.dtype], -1, COMM_REDUCE_PULL,
                             scale=(1.0 / P if avg else 1.0))
            b.add_task(int(TaskType.REDUCE_SCATTER), raw, waits=[ready], signals=[done])
            n += 1
        _close(b, [(done, n, False, False)])
        e = _store(key, _Entry([b.build()], []))
    e.programs[0].run()
    return out


def all_to_all(inp: torch.Tensor, out: torch.Tensor, in_splits: Optional[Sequence[int]] = None,
               out_splits: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Rows ``inp[in_off[d] : in_off[d] + in_splits[d]]`` go to rank d, which stores what it receives from
    rank s at ``out[out_off[s] : ...]`` (``torch.distributed.all_to_all_single`` semantics; equal splits
    when the lists are None). Both tensors live in the heap. With variable splits every sender needs
    the receiver's offset for it: the split lists are exchanged once on the host and cached per
    signature (the reference passes the lists straight to NCCL: maco/comm/nccl_ops.py:241-286)."""
    heap = _heap()
    P, r = heap.world, heap.rank
    row_bytes = inp[0].numel() * inp.element_size() if inp.dim() > 1 else inp.element_size()
    if in_splits is None:
        if inp.shape[0] % P:
            raise ValueError("all_to_all: equal splits need dim 0 divisible by world")
        in_splits = [inp.shape[0] // P] * P
        out_splits = list(in_splits)
    in_splits, out_splits = [int(v) for v in in_splits], [int(v) for v in out_splits]
    key = ("a2av", heap.offset_of(inp), heap.offset_of(out), tuple(in_splits), tuple(out_splits), row_bytes)
    e = _lookup(key)
    if e is None:
        # offset of my rows inside every destination's output = sum of that rank's out_splits before me
        if P > 1:
            from ..comm.process_group import ProcessGroupManager
            gathered = ProcessGroupManager().all_gather_object(out_splits)
        else:
            gathered = [out_splits]
        b = _builder(heap)
        ready = _open(b)
        done = b.new_event()
        src, dst = heap.offset_of(inp), heap.offset_of(out)
        in_off = 0
        n_recv = 0
        for d in range(P):
            nb = in_splits[d] * row_bytes
            if gathered[d][r] != in_splits[d]:
                raise ValueError(f"all_to_all: rank {d} expects {gathered[d][r]} rows from rank {r}, which sends {in_splits[d]}")
            d_off = sum(gathered[d][:r]) * row_bytes
            if nb % 16 or (in_off * row_bytes) % 16 or d_off % 16:
                raise ValueError("all_to_all: every block must start and end on a 16-byte boundary")
            for o, n in _chunks(nb):
                row, rows = _push_rows(n)
                raw = _pack_comm(src + in_off * row_bytes + o, dst + d_off + o, row, row, row, rows,
                                 N.DTYPE_CODE.get(inp.dtype, 0), d, COMM_PUSH)
                b.add_task(int(TaskType.ALL_TO_ALL), raw, waits=[ready], signal_peer=d, signal_peer_event=done)
            in_off += in_splits[d]
        for s_ in range(P):
            n_recv += len(list(_chunks(out_splits[s_] * row_bytes)))
        _wait_local(b, [(done, n_recv, True, False)] if n_recv else [])
        e = _store(key, _Entry([b.build()], []))
    e.programs[0].run()
    return out


def send_recv(send: Optional[torch.Tensor], dst: int, recv: Optional[torch.Tensor], src: int) -> Optional[torch.Tensor]:
    """Point-to-point put + flag: this rank's heap tensor ``send`` is written into rank ``dst``'s ``recv``
    buffer (same heap offset as this rank's ``recv``) and the receiver waits for the pieces. Ranks call it
    in matching pairs; pass None for the half a rank does not take part in. The receiver's kernel tells the
    sender that it is running before any data leaves (see the module docstring)."""
    heap = _heap()
    key = ("p2p", heap.offset_of(send) if send is not None else -1, dst, heap.offset_of(recv) if recv is not None else -1, src,
           send.numel() * send.element_size() if send is not None else 0)
    e = _lookup(key)
    if e is None:
        b = _builder(heap, workers=4)
        ready = b.new_event()           # bumped by the rank I send to; the rank I receive from waits on its own copy
        done = b.new_event()
        n_recv = 0
        if recv is not None:
            b.add_task(int(TaskType.PEER_BARRIER), b"", signal_peer=src, signal_peer_event=ready)
            n_recv = len(list(_chunks(recv.numel() * recv.element_size())))
        if send is not None:
            nbytes = send.numel() * send.element_size()
            if nbytes % 16 or recv is None:
                raise ValueError("send_recv: a multiple of 16 bytes, and the symmetric receive buffer on both sides")
            # the destination offset is that of the receive buffer, identical on every rank of a symmetric heap
            d_off = heap.offset_of(recv)
            for o, n in _chunks(nbytes):
                row, rows = _push_rows(n)
                raw = _pack_comm(heap.offset_of(send) + o, d_off + o, row, row, row, rows, N.DTYPE_CODE.get(send.dtype, 0), dst, COMM_PUSH)
                b.add_task(int(TaskType.ALLGATHER), raw, waits=[(ready, 1, True, False)], signal_peer=dst, signal_peer_event=done)
        _wait_local(b, [(done, n_recv, True, False)] if n_recv else [])
        e = _store(key, _Entry([b.build()], []))
    e.programs[0].run()
    return recv


def clear_cache() -> None:
    """Drops every cached program and staging buffer (their heap space goes with the heap: used at teardown)."""
    _cache.clear()
    _staging.clear()
