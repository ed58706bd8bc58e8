"""Collective nodes of a ``TaskGraph`` as tasks of the persistent kernel (more than one rank).

``lower_graph`` (ops/megakernel.py) calls these when the process group has more than one rank and the
symmetric heap exists. Every collective becomes communication tasks that run in the SAME launch as the
GEMM and element-wise tiles around it, waiting on row-block events of their producers and signalling
row-block events to their consumers:

* ``allgather``        pushed in 128-row chunks (multimem.st on a multicast-bound heap); a ``linear`` node that
                       reads the gathered tensor starts each tile when its 128 rows have landed
                       (all-gather -> GEMM);
* ``linear`` followed only by ``reduce_scatter``: the GEMM epilogue stores each partial tile into the owner's
                       staging slot (GEMM -> reduce-scatter, ``fused.gemm_reduce_scatter``);
* ``allreduce``        chunk owners sum (multimem.ld_reduce + multimem.st, or staged peer pushes);
* ``reduce_scatter``, ``all_to_all`` (flat and the 4-D Ulysses forms), ``broadcast``: peer pushes.

Buffers that other ranks write (gathered outputs, all-reduce targets, receive buffers) must live in the heap;
when the user's tensor does not, a heap buffer of the same size stands in and COPY tasks move the data.
The program opens with a handshake (every rank's kernel of this launch is running, hence everything the rank
queued before it has finished) and its last task waits for everything this rank receives.

The reference executes these nodes as one NCCL call each between separate kernel launches
(maco/task_graph/runtime.py:211-226).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _native as N
from ..ops.megakernel import (BM, COMM_ALLREDUCE_MC, COMM_PUSH, COMM_REDUCE_LOCAL, ProgramBuilder, RowEvents, _pack_comm)
from ..task_graph.nodes import TaskNode, TaskType
from . import fused

Wait = Tuple[int, int, bool, bool]
T_COPY = 300


class DistContext:
    """Per-program state of the multi-rank lowering."""

    def __init__(self, b: ProgramBuilder):
        self.b = b
        self.heap = b.heap
        self.rank, self.world = b.heap.rank, b.heap.world
        self.ready: Optional[Wait] = None           # opening handshake, created on first use
        self.final_waits: List[Wait] = []           # what the kernel's last task waits for
        self.heap_buffers: List[torch.Tensor] = []  # stand-ins allocated from the heap (freed with the program)

    def opening(self) -> Wait:
        if self.ready is None:
            ev = self.b.new_event()
            self.b.add_task(int(TaskType.PEER_BARRIER), b"", signal_peer=-2, signal_peer_event=ev)
            self.ready = (ev, self.world, True, False)
        return self.ready

    def merge(self, waits: Sequence[Wait]) -> Optional[Wait]:
        """One wait condition that holds when all of ``waits`` hold (a NOP task bumps a fresh event)."""
        waits = list(dict.fromkeys(waits))
        if not waits:
            return None
        if len(waits) == 1:
            return waits[0]
        ev = self.b.new_event()
        self.b.add_task(int(TaskType.NOP), b"", waits=self.b.join(waits), signals=[ev])
        return (ev, 1, False, False)

    def in_heap(self, t: torch.Tensor) -> bool:
        return self.heap.owns(t) and t.is_contiguous()

    def stand_in(self, t: torch.Tensor) -> torch.Tensor:
        buf = self.heap.alloc(tuple(t.shape), t.dtype)
        self.heap_buffers.append(buf)
        return buf

    def local_off(self, t: torch.Tensor) -> int:
        """``t``'s address as an offset from this rank's heap base (wraps for tensors outside the heap: tasks
        add it to the base in 64-bit arithmetic, which gives the address back)."""
        return (t.data_ptr() - self.heap.peer_base(self.rank)) % (1 << 64)

    def finish(self) -> None:
        """Last task: the launch ends when everything this rank receives has arrived."""
        if self.final_waits:
            self.b.add_task(int(TaskType.NOP), b"", waits=self.b.join(list(dict.fromkeys(self.final_waits))))


def _flat_rows(t: torch.Tensor) -> Tuple[int, int]:
    cols = t.shape[-1] if t.dim() else 1
    return t.numel() // max(1, cols), cols


def _copy(ctx: DistContext, src: torch.Tensor, dst: torch.Tensor, in_ready: Optional[RowEvents],
          extra: Sequence[Wait]) -> RowEvents:
    rows, cols = _flat_rows(src)
    return ctx.b.elementwise(T_COPY, src, dst, rows=rows, cols=cols, in_ready=[in_ready], extra_waits=list(extra))


def _chunks(nbytes: int, chunk: int):
    off = 0
    while off < nbytes:
        n = min(chunk, nbytes - off)
        yield off, n
        off += n


def _rows16(nbytes: int) -> Tuple[int, int]:
    row = 16384 if nbytes % 16384 == 0 else 16
    return row, nbytes // row


def can_lower_collective(node: TaskNode, heap) -> bool:
    """Shapes the tasks can express: contiguous tensors of a supported type whose blocks are whole 16-byte vectors."""
    if heap is None:
        return False
    ts = list(node.inputs) + list(node.outputs)
    if any((not x.is_contiguous()) or x.dtype not in N.DTYPE_CODE or not x.is_cuda for x in ts):
        return False
    world = heap.world
    t = node.task_type
    x = node.inputs[0]
    nbytes = x.numel() * x.element_size()
    if x.numel() == 0:
        return True
    if t == TaskType.ALLREDUCE:
        return nbytes % 16 == 0 and node.attrs.get("op", "sum") in ("sum", "avg", "mean")
    if t == TaskType.BROADCAST:
        return nbytes % 16 == 0
    if t == TaskType.ALLGATHER:
        return nbytes % 16 == 0
    if t == TaskType.REDUCE_SCATTER:
        return (nbytes // world) % 16 == 0 and node.attrs.get("op", "sum") in ("sum", "avg", "mean")
    if t == TaskType.ALL_TO_ALL:
        sd, gd = node.attrs.get("scatter_dim", 0), node.attrs.get("gather_dim", 0)
        if sd == gd == 0:
            return (nbytes // world) % 16 == 0
        if x.dim() == 4 and (sd, gd) in ((2, 1), (1, 2)):
            inner = (x.shape[2] // world if (sd, gd) == (2, 1) else x.shape[2]) * x.shape[3] * x.element_size()
            return inner % 16 == 0
        return False
    return False


def _whole(ev: RowEvents) -> Wait:
    return (ev.all_event[0], ev.all_event[1], ev.sys, False)


def _src_waits(ctx: DistContext, in_ready: Optional[RowEvents], extra: Sequence[Wait], opening: bool = True) -> List[Wait]:
    w = list(extra)
    if in_ready is not None and in_ready.all_event[1] > 0:
        w.append(_whole(in_ready))
    if opening:
        w.append(ctx.opening())
    m = ctx.merge(w)
    return [m] if m is not None else []


def lower_allgather(ctx: DistContext, node: TaskNode, in_ready: Optional[RowEvents], extra: Sequence[Wait]) -> RowEvents:
    b, heap, rank, world = ctx.b, ctx.heap, ctx.rank, ctx.world
    x, out = node.inputs[0], node.outputs[0]
    rows, cols = _flat_rows(x)
    dst = out if ctx.in_heap(out) else ctx.stand_in(out)
    if rows % BM == 0 and (cols * x.element_size()) % 16 == 0:
        fence = ctx.merge(list(extra) + [ctx.opening()])
        ev = fused.allgather_push(b, x.view(rows, cols), dst.view(world * rows, cols), fence=fence, src_ready=in_ready)
        arrivals = [(e, c, True, False) for e, c in ev.row_events if c]
    else:
        nbytes = x.numel() * x.element_size()
        waits = _src_waits(ctx, in_ready, extra)
        arr = b.new_event()
        in_place = ctx.in_heap(x) and heap.offset_of(x) == heap.offset_of(dst) + rank * nbytes
        pieces = list(_chunks(nbytes, 1 << 20))
        dests = [(rank + k) % world for k in range(1, world)] + ([] if in_place else [rank])
        for d in dests:
            for o, n in pieces:
                row, nrows = _rows16(n)
                raw = _pack_comm(ctx.local_off(x) + o, heap.offset_of(dst) + rank * nbytes + o, row, row, row, nrows,
                                 N.DTYPE_CODE[x.dtype], d, COMM_PUSH)
                b.add_task(int(TaskType.ALLGATHER), raw, waits=waits, signal_peer=d, signal_peer_event=arr, comm_worker=True)
        total = (world - (1 if in_place else 0)) * len(pieces)
        ev = RowEvents(rows=world * rows, block=BM, row_events=[], all_event=(arr, total), sys=True)
        arrivals = [(arr, total, True, False)]
        b.keepalive += [x, dst]
    ctx.final_waits += arrivals
    if dst is not out:
        if not ev.row_events:
            return _copy(ctx, dst, out, ev, [])
        # row-aligned copy out of the stand-in: each copy task waits for the block it reads
        return b.elementwise(T_COPY, dst, out, rows=world * rows, cols=cols, in_ready=[ev], rows_per_task=BM)
    return ev


def lower_reduce_scatter(ctx: DistContext, node: TaskNode, in_ready: Optional[RowEvents], extra: Sequence[Wait]) -> RowEvents:
    b, heap, rank, world = ctx.b, ctx.heap, ctx.rank, ctx.world
    x, out = node.inputs[0], node.outputs[0]
    blk = out.numel() * out.element_size()
    staging = heap.alloc((world * blk,), torch.uint8)
    ctx.heap_buffers.append(staging)
    st_off = heap.offset_of(staging)
    op = node.attrs.get("op", "sum")
    scale = 1.0 / world if op in ("avg", "mean") else 1.0
    waits = _src_waits(ctx, in_ready, extra)
    arrived, done = b.new_event(), b.new_event()
    pieces = list(_chunks(blk, 256 << 10))
    dt = N.DTYPE_CODE[x.dtype]
    for k in range(1, world + 1):
        d = (rank + k) % world                       # other ranks first, the own block last
        for o, n in pieces:
            row, nrows = _rows16(n)
            raw = _pack_comm(ctx.local_off(x) + d * blk + o, st_off + rank * blk + o, row, row, row, nrows, dt, d, COMM_PUSH)
            b.add_task(int(TaskType.REDUCE_SCATTER), raw, waits=waits, signal_peer=d, signal_peer_event=arrived,
                       comm_worker=True)
    for o, n in pieces:
        row, nrows = _rows16(n)
        raw = _pack_comm(st_off + o, 0, row, row, row, nrows, dt, -1, COMM_REDUCE_LOCAL, nslots=world, slot_stride=blk,
                         local_ptr=out.data_ptr() + o, scale=scale)
        b.add_task(int(TaskType.REDUCE_SCATTER), raw, waits=[(arrived, world * len(pieces), True, False)], signals=[done],
                   any_worker=True)
    b.keepalive += [x, out, staging]
    rows, _ = _flat_rows(out)
    return RowEvents(rows=rows, block=BM, row_events=[], all_event=(done, len(pieces)))


def fusable_linear_reduce_scatter(lin: TaskNode, rs: TaskNode, world: int) -> bool:
    """``reduce_scatter(linear(x, w))`` with nothing else reading the product: the GEMM epilogue can send the
    partial tiles straight to their owners."""
    if lin.task_type != TaskType.LINEAR or lin.attrs.get("has_bias") or lin.attrs.get("activation") not in (None, "none"):
        return False
    x, w = lin.inputs[0], lin.inputs[1]
    if x.dim() != 2 or x.dtype not in (torch.bfloat16, torch.float16) or rs.outputs[0].dtype != x.dtype:
        return False
    if rs.attrs.get("op", "sum") not in ("sum", "avg", "mean"):
        return False
    M = x.shape[0]
    return M % (world * BM) == 0 and w.shape[0] % 8 == 0 and rs.inputs[0].data_ptr() == lin.outputs[0].data_ptr()


def lower_linear_reduce_scatter(ctx: DistContext, lin: TaskNode, rs: TaskNode, a_ready: Optional[RowEvents],
                                extra: Sequence[Wait], need_opening: bool = True) -> Tuple[RowEvents, RowEvents]:
    """``need_opening`` False: the input already hangs on a collective of this launch. Whatever arrived from a peer
    left it after that peer saw every rank's opening signal, so the tiles need no opening wait of their own (a
    third condition would cost every own-block tile a join task)."""
    b, heap, world = ctx.b, ctx.heap, ctx.world
    x, w = lin.inputs[0], lin.inputs[1]
    out = rs.outputs[0]
    rows_local, Nn = x.shape[0] // world, w.shape[0]
    staging = heap.alloc((world, rows_local, Nn), x.dtype)
    ctx.heap_buffers.append(staging)
    scale = 1.0 / world if rs.attrs.get("op", "sum") in ("avg", "mean") else 1.0
    gemm_ev, out_ev = fused.gemm_reduce_scatter(b, x, w, staging, out.view(rows_local, Nn), a_ready=a_ready, scale=scale,
                                                extra_waits=list(extra) + ([ctx.opening()] if need_opening else []))
    return gemm_ev, out_ev


def lower_allreduce(ctx: DistContext, node: TaskNode, in_ready: Optional[RowEvents], extra: Sequence[Wait]) -> RowEvents:
    b, heap, rank, world = ctx.b, ctx.heap, ctx.rank, ctx.world
    t = node.inputs[0]
    scale_avg = node.attrs.get("op", "sum") in ("avg", "mean")
    buf = t if ctx.in_heap(t) else ctx.stand_in(t)
    src_extra, src_ready = list(extra), in_ready
    if buf is not t:
        src_ready = _copy(ctx, t, buf, in_ready, extra)
        src_extra = []
    nbytes = buf.numel() * buf.element_size()
    off = heap.offset_of(buf)
    dt = N.DTYPE_CODE[buf.dtype]
    if heap.multicast_base():
        # every rank announces that its copy is complete; chunk owners then reduce through the switch
        rdy, done = b.new_event(), b.new_event()
        w = _src_waits(ctx, src_ready, src_extra, opening=False)
        b.add_task(int(TaskType.PEER_BARRIER), b"", waits=w, signal_peer=-2, signal_peer_event=rdy)
        chunk = 128 << 10
        pieces = list(_chunks(nbytes, chunk))
        for c, (o, n) in enumerate(pieces):
            if c % world != rank:
                continue
            row, nrows = _rows16(n)
            raw = _pack_comm(off + o, off + o, row, row, row, nrows, dt, -1, COMM_ALLREDUCE_MC,
                             scale=(1.0 / world if scale_avg else 1.0))
            b.add_task(int(TaskType.ALLREDUCE), raw, waits=[(rdy, world, True, False)], signal_peer=-4, signal_peer_event=done,
                       comm_worker=True)
        res = (done, len(pieces))
    else:
        chunk = 256 << 10
        n_chunks = -(-nbytes // chunk)
        per_owner = -(-n_chunks // world)
        staging = heap.alloc((world * per_owner * chunk,), torch.uint8)
        ctx.heap_buffers.append(staging)
        w = _src_waits(ctx, src_ready, src_extra)
        res = fused.allreduce_push_tasks(b, buf.view(-1), staging, avg=scale_avg, chunk_bytes=chunk, fence=w[0] if w else None)
    b.keepalive.append(buf)
    ctx.final_waits.append((res[0], res[1], True, False))
    rows, _ = _flat_rows(t)
    ev = RowEvents(rows=rows, block=BM, row_events=[], all_event=res, sys=True)
    if buf is not t:
        return _copy(ctx, buf, t, ev, [])
    return ev


def lower_broadcast(ctx: DistContext, node: TaskNode, in_ready: Optional[RowEvents], extra: Sequence[Wait]) -> RowEvents:
    b, heap, rank, world = ctx.b, ctx.heap, ctx.rank, ctx.world
    t = node.inputs[0]
    src = int(node.attrs.get("src", 0))
    buf = t if ctx.in_heap(t) else ctx.stand_in(t)
    src_ready, src_extra = in_ready, list(extra)
    if buf is not t and rank == src:
        src_ready, src_extra = _copy(ctx, t, buf, in_ready, extra), []
    nbytes = buf.numel() * buf.element_size()
    off = heap.offset_of(buf)
    done = b.new_event()
    pieces = list(_chunks(nbytes, 1 << 20))
    if rank == src:
        waits = _src_waits(ctx, src_ready, src_extra)
        for o, n in pieces:
            row, nrows = _rows16(n)
            raw = _pack_comm(off + o, off + o, row, row, row, nrows, N.DTYPE_CODE.get(t.dtype, 0), -1, COMM_PUSH)
            b.add_task(int(TaskType.BROADCAST), raw, waits=waits, signal_peer=-2, signal_peer_event=done, comm_worker=True)
    else:
        ctx.opening()                                 # every rank takes part in the handshake
    b.keepalive.append(buf)
    ctx.final_waits.append((done, len(pieces), True, False))
    rows, _ = _flat_rows(t)
    ev = RowEvents(rows=rows, block=BM, row_events=[], all_event=(done, len(pieces)), sys=True)
    if buf is not t and rank != src:
        return _copy(ctx, buf, t, ev, [])
    return ev


def lower_all_to_all(ctx: DistContext, node: TaskNode, in_ready: Optional[RowEvents], extra: Sequence[Wait]) -> RowEvents:
    b, heap, rank, world = ctx.b, ctx.heap, ctx.rank, ctx.world
    x, out = node.inputs[0], node.outputs[0]
    sd, gd = node.attrs.get("scatter_dim", 0), node.attrs.get("gather_dim", 0)
    dst = out if ctx.in_heap(out) else ctx.stand_in(out)
    waits = _src_waits(ctx, in_ready, extra)
    arr = b.new_event()
    es = x.element_size()
    dt = N.DTYPE_CODE[x.dtype]
    src0, dst0 = ctx.local_off(x), heap.offset_of(dst)
    n_in = 0                                           # tasks whose data lands on this rank (same count on every rank)
    if sd == gd == 0:
        blk = x.numel() * es // world
        pieces = list(_chunks(blk, 1 << 20))
        for k in range(1, world + 1):
            d = (rank + k) % world
            for o, n in pieces:
                row, nrows = _rows16(n)
                raw = _pack_comm(src0 + d * blk + o, dst0 + rank * blk + o, row, row, row, nrows, dt, d, COMM_PUSH)
                b.add_task(int(TaskType.ALL_TO_ALL), raw, waits=waits, signal_peer=d, signal_peer_event=arr, comm_worker=True)
        n_in = world * len(pieces)
    else:
        P = world
        for k in range(1, world + 1):
            q = (rank + k) % world
            for bi in range(x.shape[0]):
                if (sd, gd) == (2, 1):                 # [B, S/P, H, D] -> [B, S, H/P, D]
                    _, s, H, D = x.shape
                    hp = H // P
                    row_bytes = hp * D * es
                    s_off = src0 + (bi * s * H * D + q * hp * D) * es
                    d_off = dst0 + (bi * s * P * hp * D + rank * s * hp * D) * es
                    nrows, s_stride, d_stride = s, H * D * es, hp * D * es
                else:                                  # [B, S, H/P, D] -> [B, S/P, H, D]
                    _, S, h, D = x.shape
                    sp = S // P
                    row_bytes = h * D * es
                    s_off = src0 + (bi * S * h * D + q * sp * h * D) * es
                    d_off = dst0 + (bi * sp * P * h * D + rank * h * D) * es
                    nrows, s_stride, d_stride = sp, h * D * es, P * h * D * es
                raw = _pack_comm(s_off, d_off, s_stride, d_stride, row_bytes, nrows, dt, q, COMM_PUSH)
                b.add_task(int(TaskType.ALL_TO_ALL), raw, waits=waits, signal_peer=q, signal_peer_event=arr, comm_worker=True)
        n_in = world * x.shape[0]
    b.keepalive += [x, dst]
    ctx.final_waits.append((arr, n_in, True, False))
    rows, _ = _flat_rows(out)
    ev = RowEvents(rows=rows, block=BM, row_events=[], all_event=(arr, n_in), sys=True)
    if dst is not out:
        return _copy(ctx, dst, out, ev, [])
    return ev
