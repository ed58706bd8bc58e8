"""Stand-alone collectives served by the persistent kernel's communication tasks.

Each call builds (once, then caches) a small program over a buffer of the symmetric heap and
launches it: all ranks' kernels pull / push over NVLink peer memory and synchronise through
event counters in the heap. These back ``comm.patterns`` when ``config.backend == "peer"``, and
the ``nvshmem_*`` compatibility calls. NCCL stays available as the baseline (``comm.nccl_ops``).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch

from .. import _native as N
from ..ops.megakernel import COMM_PUSH, COMM_REDUCE_PULL, Program, ProgramBuilder, _pack_comm
from ..task_graph.nodes import TaskType
from . import fused
from .symm_heap import current_heap

_cache: Dict[tuple, Program] = {}
_scratch: Dict[tuple, torch.Tensor] = {}


def _heap():
    h = current_heap()
    if h is None:
        raise RuntimeError("the symmetric heap is not initialised; call maco_b200.init_nvshmem() / init()")
    return h


def _builder(heap, workers: int = 16) -> ProgramBuilder:
    return ProgramBuilder(heap.device, num_workers=workers, mode="static", heap=heap)


def all_reduce(t: torch.Tensor, avg: bool = False) -> torch.Tensor:
    """In-place sum (or mean) of heap tensor ``t`` over all ranks."""
    heap = _heap()
    key = ("ar", heap.offset_of(t), t.numel(), t.dtype, avg)
    prog = _cache.get(key)
    if prog is None:
        nbytes = t.numel() * t.element_size()
        chunk = 256 << 10
        n_chunks = -(-nbytes // chunk)
        per_owner = -(-n_chunks // heap.world)
        # staging of its own per program: two programs sharing it could overlap across ranks (each program's
        # fence only orders its own launches)
        staging = _scratch[("ar_stage",) + key] = heap.alloc((heap.world * per_owner * chunk,), torch.uint8)
        b = _builder(heap, workers=max(1, min(32, nbytes >> 18)))
        fence = fused.epoch_fence_event(b)
        done, n = fused.allreduce_push_tasks(b, t.view(-1), staging, avg=avg, chunk_bytes=chunk, fence=fence)
        fused.epoch_fence_signal(b, [(done, n, True, False)])
        prog = _cache[key] = b.build()
    prog.run()
    return t


def _scratch_like(t: torch.Tensor, tag: str, shape=None) -> torch.Tensor:
    heap = _heap()
    shape = tuple(shape if shape is not None else t.shape)
    key = (tag, shape, t.dtype)
    buf = _scratch.get(key)
    if buf is None:
        buf = _scratch[key] = heap.alloc(shape, t.dtype)
    return buf


def all_reduce_any(t: torch.Tensor, avg: bool = False) -> torch.Tensor:
    """All-reduce of any CUDA tensor: staged through a heap buffer when ``t`` lives outside the heap."""
    heap = _heap()
    if heap.owns(t) and t.is_contiguous():
        return all_reduce(t, avg)
    if t.dtype not in N.DTYPE_CODE:
        raise ValueError(f"unsupported dtype {t.dtype}")
    numel = (t.numel() * t.element_size() + 15) // 16 * 16 // t.element_size()
    buf = _scratch_like(t, "ar", (numel,))
    buf.zero_()
    buf[: t.numel()].copy_(t.reshape(-1))
    all_reduce(buf, avg)
    t.copy_(buf[: t.numel()].view(t.shape))
    return t


def device_barrier() -> None:
    """All ranks' kernels meet: each bumps every rank's counter and waits for ``world`` bumps."""
    heap = _heap()
    key = ("barrier",)
    prog = _cache.get(key)
    if prog is None:
        b = _builder(heap, workers=1)
        ev = b.new_event()
        b.add_task(int(TaskType.PEER_BARRIER), b"", signal_peer=-2, signal_peer_event=ev)
        b.add_task(int(TaskType.NOP), b"", waits=[(ev, heap.world, True, False)])
        prog = _cache[key] = b.build()
    prog.run()


def all_gather(shard: torch.Tensor, gathered: torch.Tensor) -> torch.Tensor:
    """``gathered`` [world*rows, cols] <- every rank's ``shard`` [rows, cols]; both in the heap."""
    heap = _heap()
    key = ("ag", heap.offset_of(shard), heap.offset_of(gathered), tuple(shard.shape), shard.dtype)
    prog = _cache.get(key)
    if prog is None:
        b = _builder(heap)
        fence = fused.epoch_fence_event(b)
        ev = fused.allgather_push(b, shard, gathered, fence=fence)
        waits = b.join([(e, c, True, False) for e, c in ev.row_events])
        fused.epoch_fence_signal(b, waits)
        prog = _cache[key] = b.build()
    prog.run()
    return gathered


def all_to_all_4d(t: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1) -> torch.Tensor:
    """Ulysses layout switch on a heap tensor, written straight into the destination layout:
    (2,1): [B, S/P, H, D] -> [B, S, H/P, D];  (1,2): [B, S, H/P, D] -> [B, S/P, H, D].
    Each (batch, sequence position, destination rank) slice is one row of a strided 2-D push, so
    there are no pack / unpack passes (the reference packs, exchanges and unpacks:
    maco/comm/patterns.py:400-436, maco/csrc/nvshmem_ops.cu:399-494)."""
    heap = _heap()
    P, r = heap.world, heap.rank
    if (scatter_dim, gather_dim) == (2, 1):
        B, s, H, D = t.shape
        out_shape = (B, s * P, H // P, D)
    elif (scatter_dim, gather_dim) == (1, 2):
        B, S, h, D = t.shape
        out_shape = (B, S // P, h * P, D)
    else:
        raise ValueError("all_to_all_4d supports (scatter, gather) = (2, 1) or (1, 2)")
    out = _scratch_like(t, f"a2a{scatter_dim}{gather_dim}", out_shape)
    key = ("a2a", heap.offset_of(t), heap.offset_of(out), tuple(t.shape), t.dtype, scatter_dim, gather_dim)
    prog = _cache.get(key)
    if prog is None:
        b = _builder(heap)
        fence = fused.epoch_fence_event(b)
        done = b.new_event()
        es = t.element_size()
        src, dst = heap.offset_of(t), heap.offset_of(out)
        n_tasks = 0
        for q in range(P):
            for bi in range(t.shape[0]):
                if (scatter_dim, gather_dim) == (2, 1):
                    hp = H // P
                    row_bytes = hp * D * es                      # the heads rank q keeps, for one position
                    s_off = src + (bi * s * H * D + q * hp * D) * es
                    d_off = dst + (bi * s * P * hp * D + r * s * hp * D) * es
                    rows, s_stride, d_stride = s, H * D * es, hp * D * es
                else:
                    sp = S // P
                    row_bytes = h * D * es
                    s_off = src + (bi * S * h * D + q * sp * h * D) * es
                    d_off = dst + (bi * sp * P * h * D + r * h * D) * es
                    rows, s_stride, d_stride = sp, h * D * es, P * h * D * es
                raw = _pack_comm(s_off, d_off, s_stride, d_stride, row_bytes, rows, N.DTYPE_CODE[t.dtype], q, COMM_PUSH)
                b.add_task(int(TaskType.ALL_TO_ALL), raw, waits=[fence], signal_peer=q, signal_peer_event=done)
                n_tasks += 1
        fused.epoch_fence_signal(b, [(done, n_tasks, True, False)])
        prog = _cache[key] = b.build()
    prog.run()
    return out


def all_to_all_4d_any(t: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1) -> torch.Tensor:
    heap = _heap()
    if not (heap.owns(t) and t.is_contiguous()):
        buf = _scratch_like(t, "a2a_in")
        buf.copy_(t)
        t = buf
    return all_to_all_4d(t, scatter_dim, gather_dim).clone()


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
    prog = _cache.get(key)
    if prog is None:
        b = _builder(heap)
        fence = fused.epoch_fence_event(b)
        done = b.new_event()
        off = heap.offset_of(t)
        pieces = list(_chunks(nbytes))
        if heap.rank == src:
            for o, n in pieces:
                row, rows = _push_rows(n)
                raw = _pack_comm(off + o, off + o, row, row, row, rows, N.DTYPE_CODE.get(t.dtype, 0), -1, COMM_PUSH)
                b.add_task(int(TaskType.BROADCAST), raw, waits=[fence], signal_peer=-2, signal_peer_event=done)
        fused.epoch_fence_signal(b, [(done, len(pieces), True, False)])
        prog = _cache[key] = b.build()
    prog.run()
    return t


def reduce_scatter(inp: torch.Tensor, out: torch.Tensor, avg: bool = False) -> torch.Tensor:
    """``out`` [rows, ...] <- sum over ranks of block ``rank`` of their ``inp`` [world*rows, ...]; both in
    the heap. Every rank pulls its block from all ranks over NVLink and sums in fp32."""
    heap = _heap()
    P, r = heap.world, heap.rank
    nbytes = out.numel() * out.element_size()
    if inp.numel() != out.numel() * P or nbytes % 16 or inp.dtype != out.dtype:
        raise ValueError("reduce_scatter: inp must hold world blocks of out's size (a multiple of 16 bytes)")
    key = ("rs", heap.offset_of(inp), heap.offset_of(out), nbytes, out.dtype, avg)
    prog = _cache.get(key)
    if prog is None:
        b = _builder(heap)
        fence = fused.epoch_fence_event(b)
        ready = b.new_event()
        b.add_task(int(TaskType.NOP), b"", waits=[fence], signal_peer=-2, signal_peer_event=ready)
        done = b.new_event()
        src, dst = heap.offset_of(inp) + r * nbytes, heap.offset_of(out)
        n = 0
        for o, nb in _chunks(nbytes, 256 << 10):
            row, rows = _push_rows(nb)
            raw = _pack_comm(src + o, dst + o, row, row, row, rows, N.DTYPE_CODE[out.dtype], -1, COMM_REDUCE_PULL,
                             scale=(1.0 / P if avg else 1.0))
            b.add_task(int(TaskType.REDUCE_SCATTER), raw, waits=[(ready, P, True, False)], signals=[done])
            n += 1
        fused.epoch_fence_signal(b, [(done, n, False, False)])
        prog = _cache[key] = b.build()
    prog.run()
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
    prog = _cache.get(key)
    if prog is None:
        # offset of my rows inside every destination's output = sum of that rank's out_splits before me
        if P > 1:
            from ..comm.process_group import ProcessGroupManager
            gathered = ProcessGroupManager().all_gather_object(out_splits)
        else:
            gathered = [out_splits]
        b = _builder(heap)
        fence = fused.epoch_fence_event(b)
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
                b.add_task(int(TaskType.ALL_TO_ALL), raw, waits=[fence], signal_peer=d, signal_peer_event=done)
            in_off += in_splits[d]
        for s_ in range(P):
            n_recv += len(list(_chunks(out_splits[s_] * row_bytes)))
        fused.epoch_fence_signal(b, [(done, n_recv, True, False)] if n_recv else [])
        prog = _cache[key] = b.build()
    prog.run()
    return out


def send_recv(send: Optional[torch.Tensor], dst: int, recv: Optional[torch.Tensor], src: int) -> Optional[torch.Tensor]:
    """Point-to-point put + flag: this rank's heap tensor ``send`` is written into rank ``dst``'s ``recv``
    buffer (same heap offset as this rank's ``recv``) and the receiver waits for the pieces. Ranks call it
    in matching pairs; pass None for the half a rank does not take part in."""
    heap = _heap()
    key = ("p2p", heap.offset_of(send) if send is not None else -1, dst, heap.offset_of(recv) if recv is not None else -1, src,
           send.numel() * send.element_size() if send is not None else 0)
    prog = _cache.get(key)
    if prog is None:
        b = _builder(heap, workers=4)
        fence = fused.epoch_fence_event(b)
        done = b.new_event()
        n_recv = 0
        if send is not None:
            nbytes = send.numel() * send.element_size()
            if nbytes % 16 or recv is None:
                raise ValueError("send_recv: a multiple of 16 bytes, and the symmetric receive buffer on both sides")
            # the destination offset is that of the receive buffer, identical on every rank of a symmetric heap
            d_off = heap.offset_of(recv)
            for o, n in _chunks(nbytes):
                row, rows = _push_rows(n)
                raw = _pack_comm(heap.offset_of(send) + o, d_off + o, row, row, row, rows, N.DTYPE_CODE.get(send.dtype, 0), dst, COMM_PUSH)
                b.add_task(int(TaskType.ALLGATHER), raw, waits=[fence], signal_peer=dst, signal_peer_event=done)
        if recv is not None:
            n_recv = len(list(_chunks(recv.numel() * recv.element_size())))
        fused.epoch_fence_signal(b, [(done, n_recv, True, False)] if n_recv else [])
        prog = _cache[key] = b.build()
    prog.run()
    return recv


def clear_cache() -> None:
    _cache.clear()
    _scratch.clear()
