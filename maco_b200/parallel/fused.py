"""Fused compute + collective task patterns for the persistent kernel.

Each helper appends tasks to a ``ProgramBuilder`` so that the transfer over NVLink overlaps the
tensor-core tiles inside ONE kernel, tile by tile:

* ``allgather_push``        shard rows are pushed into every rank's gathered buffer in chunks; each
                            128-row block of the gathered buffer has its own event, so a GEMM tile
                            starts as soon as the rows it reads have landed (all-gather -> GEMM).
* ``gemm_reduce_scatter``   the GEMM epilogue stores each partial tile straight into the staging slot
                            of the rank that owns those rows and bumps that rank's per-block counter;
                            the owner sums the slots when the counter is full, or, with two ranks,
                            adds the peer's slot in the epilogue of its own tiles (GEMM -> reduce-scatter).
* ``gemm_allreduce``        few-row GEMM as split-K tiles whose finishing tasks store the partial rows
                            into every rank's slot; each rank sums its slots plus the residual.
* ``allreduce_tasks``       two-shot all-reduce in chunks: the chunk's owner pulls it from every rank,
                            reduces in fp32 and writes the result back to every rank.
* ``epoch_fence``           end-of-launch signal that keeps a faster rank's next launch from
                            overwriting buffers a slower rank still reads.

The reference has no such path: its tensor-parallel example all-reduces a column-parallel output
(examples/tensor_parallel.py:55-61) and every collective is a separate NCCL call.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .. import _native as N
from ..ops.megakernel import (BM, COMM_ALLREDUCE, COMM_PUSH, COMM_PUSH_MC, COMM_REDUCE_LOCAL, COMM_REDUCE_LOCAL_BCAST,
                              ProgramBuilder, RowEvents, _pack_comm)
from ..task_graph.nodes import TaskType


def epoch_fence_event(b: ProgramBuilder) -> Tuple[int, int, bool, bool]:
    """Allocates the cross-rank "previous launch finished everywhere" condition: an event every
    rank bumps once at the end of a launch; waited on with the previous epoch's threshold."""
    ev = b.new_event()
    b._fence_event = ev
    return (ev, b.heap.world, True, True)


def epoch_fence_signal(b: ProgramBuilder, waits: Sequence[Tuple[int, int, bool, bool]]) -> None:
    """Final task of a program: when ``waits`` hold, tell every rank this rank is done."""
    waits = b.join(list(waits))
    b.add_task(int(TaskType.NOP), b"", waits=waits, signal_peer=-2, signal_peer_event=b._fence_event)


def allgather_push(b: ProgramBuilder, shard: torch.Tensor, gathered: torch.Tensor, *, chunk_rows: int = 128,
                   fence: Optional[Tuple[int, int, bool, bool]] = None,
                   src_ready: Optional[RowEvents] = None, multicast: Optional[bool] = None) -> RowEvents:
    """Pushes this rank's ``shard`` [rows, cols] into rows ``[rank*rows, (rank+1)*rows)`` of every
    rank's ``gathered`` [world*rows, cols]. Returns row-block events of ``gathered``.

    ``shard`` may BE that slice of this rank's ``gathered`` (no local copy is made then, and the
    local blocks carry an always-true condition). With plain peer memory: one task per (destination,
    chunk), ordered by when the destination needs the rows (rank r-1 consumes this shard first, then
    r-2, ...). ``multicast=True`` (needs a multicast-bound heap): one task per chunk stores the rows ONCE to
    the NVSwitch multicast address (multimem.st) and bumps the block's counter on every rank with one
    multimem.red; the shard leaves the GPU once instead of world-1 times, and every rank receives block j of
    every shard at about the same time (see ``gathered_order``). It is opt-in: the 128 general threads of a
    worker reach about 3 GB/s with 16-byte multimem.st (2 GPUs, measured), against 11-17 GB/s per worker for
    the bulk-copy engine's peer stores, so the multicast form only pays with many destinations.
    """
    heap = b.heap
    rank, world = heap.rank, heap.world
    rows, cols = shard.shape
    if rows % BM:
        raise ValueError("all-gather shards must be a multiple of 128 rows")
    if BM % chunk_rows:
        raise ValueError("chunk_rows must divide 128")
    row_bytes = cols * shard.element_size()
    # the source is read by this rank only: it may live outside the heap (its offset from the heap base then wraps)
    g_off = heap.offset_of(gathered)
    s_off = heap.offset_of(shard) if heap.owns(shard) else (shard.data_ptr() - heap.peer_base(rank)) % (1 << 64)
    in_place = heap.owns(shard) and s_off == g_off + rank * rows * row_bytes
    blocks = world * rows // BM
    events = [b.new_event() for _ in range(blocks)]
    all_ev = b.new_event()
    per_block = BM // chunk_rows
    multicast = bool(multicast)
    if multicast and not heap.multicast_base():
        raise ValueError("the symmetric heap has no multicast binding")
    if multicast:
        for c0 in range(0, rows, chunk_rows):
            waits = []
            if fence is not None:
                waits.append(fence)
            if src_ready is not None:
                ev, cnt = src_ready.for_rows(c0, c0 + chunk_rows)
                waits.append((ev, cnt, src_ready.sys, False))
            grow = rank * rows + c0
            raw = _pack_comm(s_off + c0 * row_bytes, g_off + grow * row_bytes, row_bytes, row_bytes, row_bytes,
                             chunk_rows, N.DTYPE_CODE[shard.dtype], -1, COMM_PUSH_MC)
            b.add_task(int(TaskType.ALLGATHER), raw, waits=waits, signal_peer=-4, signal_peer_event=events[grow // BM],
                       comm_worker=True)
        b.keepalive += [shard, gathered]
        own = range(rank * rows // BM, (rank + 1) * rows // BM)
        # the multicast store also lands in this rank's own copy: its blocks are counted like everybody's unless
        # they are already in place
        row_events = [(e, 0 if (in_place and i in own) else per_block) for i, e in enumerate(events)]
        return RowEvents(rows=world * rows, block=BM, row_events=row_events, all_event=(all_ev, 0), sys=True)
    dests = [(rank - k) % world for k in range(1, world)]
    if not in_place:
        # The local copy goes first and through the communication workers' bulk copies. (On the compute workers,
        # whose operand rings are busy, it would run as plain vector loads and stores: measured 500 us slower
        # for the 2-GPU TP MLP.)
        dests = [rank] + dests
    for dst in dests:
        for c0 in range(0, rows, chunk_rows):
            waits = []
            if fence is not None:
                waits.append(fence)
            if src_ready is not None:
                ev, cnt = src_ready.for_rows(c0, c0 + chunk_rows)
                waits.append((ev, cnt, src_ready.sys, False))
            grow = rank * rows + c0
            raw = _pack_comm(s_off + c0 * row_bytes, g_off + grow * row_bytes, row_bytes, row_bytes, row_bytes,
                             chunk_rows, N.DTYPE_CODE[shard.dtype], dst, COMM_PUSH)
            b.add_task(int(TaskType.ALLGATHER), raw, waits=waits, signal_peer=dst, signal_peer_event=events[grow // BM],
                       comm_worker=True)
    b.keepalive += [shard, gathered]
    own = range(rank * rows // BM, (rank + 1) * rows // BM)
    row_events = [(e, 0 if (in_place and i in own) else per_block) for i, e in enumerate(events)]
    return RowEvents(rows=world * rows, block=BM, row_events=row_events, all_event=(all_ev, 0), sys=True)


def gathered_order(rank: int, world: int, blocks_per_rank: int, multicast: bool) -> List[int]:
    """Order in which a rank consumes the row blocks of an all-gathered buffer. Peer pushes deliver shard
    rank+1 first, then rank+2, ... (``rotated_blocks``). Multicast stores deliver block j of EVERY shard at
    about the same time: own shard first, then block 0 of all other shards, block 1 of all, ..."""
    if not multicast:
        return rotated_blocks(rank, world, blocks_per_rank)
    out = list(range(rank * blocks_per_rank, (rank + 1) * blocks_per_rank))
    for j in range(blocks_per_rank):
        out += [((rank + k) % world) * blocks_per_rank + j for k in range(1, world)]
    return out


def rotated_blocks(rank: int, world: int, blocks_per_rank: int, own_last: bool = False) -> List[int]:
    """Row blocks ordered own shard first, then rank+1, rank+2, ... (the order gathered rows arrive
    in); with ``own_last`` the own shard comes last (partial results for other owners leave first, and
    the owner's reduction of a block can start right after its own tile of that block). Either way the
    ranks talk to different peers at any moment."""
    out: List[int] = []
    ks = list(range(1, world)) + [0] if own_last else list(range(world))
    for k in ks:
        r = (rank + k) % world
        out += list(range(r * blocks_per_rank, (r + 1) * blocks_per_rank))
    return out


# Up to this many ranks the own tiles of a fused GEMM -> reduce-scatter sum the peers' slots in their epilogue; beyond
# it reduction tasks spread over every worker do the sums. Two ranks: one slot, always there in time. The several-slot
# form (``aux_slots`` of the residual epilogue) works and is tested at four ranks, but measured slower there for the
# 8192 x 4096 x 14336 layer (651 us against 618-628 us with reduction tasks): the own tiles wait for the slowest
# peer's partial and their epilogues read three 64 KB slots with plain loads, which stretches the tiles of the
# last phase by more than the 40 us tail of reduction tasks it removes.
EPILOGUE_REDUCE_MAX_WORLD = 2           # the environment variable MACO_EPILOGUE_REDUCE_MAX_WORLD (2..4) overrides it


def gemm_reduce_scatter(b: ProgramBuilder, a: torch.Tensor, w: torch.Tensor, staging: torch.Tensor,
                        out: torch.Tensor, *, a_ready: Optional[RowEvents] = None, bn: int = 256,
                        reduce_rows: Optional[int] = None, scale: float = 1.0,
                        extra_waits: Sequence[Tuple[int, int, bool, bool]] = ()) -> Tuple[RowEvents, RowEvents]:
    """``out[rows_local, N] = reduce_scatter(a @ w.T)`` with the partial tiles leaving through the
    GEMM epilogue. ``staging`` is a heap tensor [world, rows_local, N] (slot = source rank).

    Tiles of row blocks owned by other ranks go straight into the owner's slot (bulk stores from the
    epilogue) and bump the owner's per-block counter; the own row blocks are computed last.
    Two ranks: by then the peer's partial for them has arrived (each rank serves the other first), so
    the own tile's epilogue adds the peer's slot to its accumulator and writes the final rows; no
    reduction pass runs after the last GEMM tile. More ranks: the last peer delivers only when the own
    blocks start, so the own tiles go to the local slot and the owner sums the slots with short
    bulk-staged tasks spread over every worker (all of them are idle by then).
    Returns (events of the GEMM tiles, events of ``out``)."""
    heap = b.heap
    rank, world = heap.rank, heap.world
    M, K = a.shape
    Nn = w.shape[0]
    rows_local = M // world
    if M % (world * BM):
        raise ValueError("rows must be a multiple of world * 128")
    blocks_per_rank = rows_local // BM
    n_tiles = (Nn + bn - 1) // bn
    es = staging.element_size()
    st_off = heap.offset_of(staging)
    slot_bytes = rows_local * Nn * es
    row_bytes = Nn * es
    part_events = [b.new_event() for _ in range(blocks_per_rank)]
    order = rotated_blocks(rank, world, blocks_per_rank, own_last=True)
    if world == 2 and scale == 1.0:
        own_first = rank * blocks_per_rank
        shift = rank * rows_local          # epilogue rows are the tile's global rows: shift both bases back
        epi_own = b.add_epilogue(out.data_ptr() - shift * out.stride(0) * out.element_size(), out.stride(0), out.dtype, M, Nn,
                                 mode="residual", aux_ptr=staging[1 - rank].data_ptr() - shift * row_bytes, ld_aux=Nn,
                                 aux_dtype=staging.dtype)

        def per_tile2(mb: int, nb: int) -> dict:
            owner = mb // blocks_per_rank
            if owner == rank:
                return dict(epi=epi_own, waits=[(part_events[mb - own_first], n_tiles, True, False)])
            return dict(peer=owner, out_off=st_off + rank * slot_bytes, row_off=-(owner * rows_local), signal_peer=owner,
                        signal_peer_event=part_events[mb % blocks_per_rank])

        gemm_ev = b.gemm(a, w, staging[0], a_ready=a_ready, bn=bn, per_tile=per_tile2, m_blocks=order, extra_waits=extra_waits)
        b.keepalive += [staging, out]
        own = gemm_ev.row_events[own_first: own_first + blocks_per_rank]
        return gemm_ev, RowEvents(rows=rows_local, block=BM, row_events=list(own), all_event=gemm_ev.all_event)

    import os
    if world <= int(os.environ.get("MACO_EPILOGUE_REDUCE_MAX_WORLD", EPILOGUE_REDUCE_MAX_WORLD)) and scale == 1.0:
        # Three or four ranks: the same idea with several slots. Rank r serves the owners r+1, r+2, ... in turn and
        # its own blocks last, so the last peer's partial for block j of this rank left one phase before this rank
        # reaches block j; the own tile's epilogue adds the world-1 peer slots to its accumulator (a few microseconds
        # of loads per tile, hidden under the next tile's main loop) and no reduction tasks follow the last tile.
        # (With reduction tasks, 4 GPUs: 256 tasks queued behind the tiles run as two rounds of 18 us.)
        own_first = rank * blocks_per_rank
        shift = rank * rows_local
        epi_own = b.add_epilogue(out.data_ptr() - shift * out.stride(0) * out.element_size(), out.stride(0), out.dtype, M, Nn,
                                 mode="residual", aux_ptr=staging[0].data_ptr() - shift * row_bytes, ld_aux=Nn,
                                 aux_dtype=staging.dtype, aux_slots=(world, rank, rows_local))

        def per_tile_n(mb: int, nb: int) -> dict:
            owner = mb // blocks_per_rank
            if owner == rank:
                return dict(epi=epi_own, waits=[(part_events[mb - own_first], (world - 1) * n_tiles, True, False)])
            return dict(peer=owner, out_off=st_off + rank * slot_bytes, row_off=-(owner * rows_local), signal_peer=owner,
                        signal_peer_event=part_events[mb % blocks_per_rank])

        gemm_ev = b.gemm(a, w, staging[0], a_ready=a_ready, bn=bn, per_tile=per_tile_n, m_blocks=order, extra_waits=extra_waits)
        b.keepalive += [staging, out]
        own = gemm_ev.row_events[own_first: own_first + blocks_per_rank]
        return gemm_ev, RowEvents(rows=rows_local, block=BM, row_events=list(own), all_event=gemm_ev.all_event)

    if reduce_rows is None:
        # about one reduction task per worker, so the tail after the last GEMM tile is one short task
        reduce_rows = 4
        while reduce_rows * 2 <= BM and rows_local // (reduce_rows * 2) >= b.num_workers:
            reduce_rows *= 2

    def per_tile(mb: int, nb: int) -> dict:
        owner = mb // blocks_per_rank
        return dict(peer=owner, out_off=st_off + rank * slot_bytes, row_off=-(owner * rows_local), signal_peer=owner,
                    signal_peer_event=part_events[mb % blocks_per_rank])

    gemm_ev = b.gemm(a, w, staging[0], a_ready=a_ready, bn=bn, per_tile=per_tile, m_blocks=order, extra_waits=extra_waits)
    # owner-side reduction of the `world` slots, fp32 accumulation
    out_events = [b.new_event() for _ in range(blocks_per_rank)]
    all_ev = b.new_event()
    total = 0
    for j in range(blocks_per_rank):
        for r0 in range(j * BM, (j + 1) * BM, reduce_rows):
            raw = _pack_comm(st_off + r0 * row_bytes, 0, row_bytes, row_bytes, row_bytes, reduce_rows,
                             N.DTYPE_CODE[staging.dtype], -1, COMM_REDUCE_LOCAL, nslots=world, slot_stride=slot_bytes,
                             local_ptr=out.data_ptr() + r0 * out.stride(0) * out.element_size(), scale=scale)
            b.add_task(int(TaskType.REDUCE_SCATTER), raw, waits=[(part_events[j], world * n_tiles, True, False)],
                       signals=[out_events[j], all_ev], any_worker=True)
            total += 1
    b.keepalive += [staging, out]
    per_block = BM // reduce_rows
    return gemm_ev, RowEvents(rows=rows_local, block=BM, row_events=[(e, per_block) for e in out_events],
                              all_event=(all_ev, total))


def allreduce_tasks(b: ProgramBuilder, buf: torch.Tensor, *, avg: bool = False, chunk_bytes: int = 1 << 20,
                    ready_waits: Sequence[Tuple[int, int, bool, bool]] = (),
                    ready_event: Optional[int] = None, comm_worker: bool = True) -> Tuple[int, int]:
    """In-place all-reduce of heap tensor ``buf`` in chunks. Chunk c is owned by rank c % world, which
    pulls it from every rank, reduces and writes it back everywhere. ``ready_event`` (bumped once
    by every rank when its data is complete) gates the pulls; when None a NOP task with
    ``ready_waits`` announces readiness. Returns (completion event, count) local to every rank."""
    heap = b.heap
    rank, world = heap.rank, heap.world
    nbytes = buf.numel() * buf.element_size()
    if nbytes % 16:
        raise ValueError("all-reduce buffers must be a multiple of 16 bytes")
    off = heap.offset_of(buf)
    if ready_event is None:
        ready_event = b.new_event()
        b.add_task(int(TaskType.NOP), b"", waits=b.join(list(ready_waits)), signal_peer=-2, signal_peer_event=ready_event)
    done = b.new_event()
    row = 16384 if nbytes >= 16384 and nbytes % 16384 == 0 else 16
    chunk_bytes = max(row, chunk_bytes // row * row)
    n_chunks = (nbytes + chunk_bytes - 1) // chunk_bytes
    for c in range(n_chunks):
        if c % world != rank:
            continue
        c0 = c * chunk_bytes
        cb = min(chunk_bytes, nbytes - c0)
        raw = _pack_comm(off + c0, off + c0, row, row, row, cb // row, N.DTYPE_CODE[buf.dtype], -1, COMM_ALLREDUCE,
                         scale=(1.0 / world if avg else 1.0))
        b.add_task(int(TaskType.ALLREDUCE), raw, waits=[(ready_event, world, True, False)], signal_peer=-2,
                   signal_peer_event=done, comm_worker=comm_worker)
    b.keepalive.append(buf)
    return done, n_chunks


def allreduce_push_tasks(b: ProgramBuilder, buf: torch.Tensor, staging: torch.Tensor, *, avg: bool = False,
                         chunk_bytes: int = 256 << 10,
                         fence: Optional[Tuple[int, int, bool, bool]] = None) -> Tuple[int, int]:
    """In-place all-reduce of heap tensor ``buf`` without remote reads (one SM reads a peer's memory
    several times slower than it writes it). Chunk c belongs to rank c % world: every rank stores its
    copy of the chunk into slot ``rank`` of the owner's ``staging`` ([world, ceil(chunks / world) *
    chunk_bytes] bytes, in the heap), the owner sums the ``world`` local slots in fp32 and stores the
    result into ``buf`` on every rank. Returns (completion event, count) local to every rank."""
    heap = b.heap
    rank, world = heap.rank, heap.world
    nbytes = buf.numel() * buf.element_size()
    if nbytes % 16:
        raise ValueError("all-reduce buffers must be a multiple of 16 bytes")
    off, st_off = heap.offset_of(buf), heap.offset_of(staging)
    row = 16384 if chunk_bytes % 16384 == 0 and nbytes % 16384 == 0 else 16
    chunk_bytes = max(row, chunk_bytes // row * row)
    n_chunks = (nbytes + chunk_bytes - 1) // chunk_bytes
    per_owner = (n_chunks + world - 1) // world
    slot_bytes = per_owner * chunk_bytes
    if staging.numel() * staging.element_size() < world * slot_bytes:
        raise ValueError("all-reduce staging buffer too small")
    done = b.new_event()
    dt = N.DTYPE_CODE[buf.dtype]
    for c in range(n_chunks):
        owner, j = c % world, c // world
        c0 = c * chunk_bytes
        cb = min(chunk_bytes, nbytes - c0)
        arrived = b.new_event()
        raw = _pack_comm(off + c0, st_off + rank * slot_bytes + j * chunk_bytes, row, row, row, cb // row, dt, owner, COMM_PUSH)
        b.add_task(int(TaskType.ALLREDUCE), raw, waits=[fence] if fence is not None else [], signal_peer=owner,
                   signal_peer_event=arrived)
        if owner == rank:
            raw = _pack_comm(st_off + j * chunk_bytes, off + c0, row, row, row, cb // row, dt, -1, COMM_REDUCE_LOCAL_BCAST,
                             nslots=world, slot_stride=slot_bytes, scale=(1.0 / world if avg else 1.0))
            b.add_task(int(TaskType.ALLREDUCE), raw, waits=[(arrived, world, True, False)], signal_peer=-2,
                       signal_peer_event=done)
    b.keepalive += [buf, staging]
    return done, n_chunks


def gemm_allreduce(b: ProgramBuilder, a: torch.Tensor, w: torch.Tensor, slots: Optional[torch.Tensor],
                   out: torch.Tensor, *, residual: Optional[torch.Tensor] = None, a_ready: Optional[RowEvents] = None,
                   extra_waits: Sequence[Tuple[int, int, bool, bool]] = (), bn: int = 128,
                   reduce_rows: Optional[int] = None, w_blocked: Optional[torch.Tensor] = None) -> RowEvents:
    """``out = all_reduce(a @ w.T) (+ residual)`` for small row counts (decode): the GEMM epilogue stores
    every partial tile into slot ``rank`` of ALL ranks' ``slots`` [world, M, N] (one-shot exchange) and
    bumps their counters; each rank then sums its slots and the residual. With one rank the residual is
    added in the GEMM epilogue and nothing is exchanged. ``w_blocked``: ``ops.block_weight(w)`` for the split-K form."""
    M, Nn = a.shape[0], w.shape[0]
    heap = b.heap
    splitk = M <= BM and Nn % 256 == 0 and a.shape[1] % 64 == 0 and (residual is None or residual.stride(0) == out.stride(0))
    if heap is None or heap.world == 1:
        if splitk:
            return b.gemm_splitk(a, w, out, epilogue="residual" if residual is not None else None, aux=residual,
                                 a_ready=a_ready, extra_waits=extra_waits, w_blocked=w_blocked)
        return b.gemm(a, w, out, epilogue="residual" if residual is not None else None, aux=residual, a_ready=a_ready,
                      extra_waits=extra_waits, bn=bn)
    rank, world = heap.rank, heap.world
    if M > BM:
        raise ValueError("gemm_allreduce is the one-shot form for at most 128 rows")
    off = heap.offset_of(slots)
    slot_bytes = M * Nn * slots.element_size()
    arrived = b.new_event()
    if splitk:
        # split-K tiles over every SM; the finishing tasks write this rank's partial into slot `rank` of every rank
        fin = b.gemm_splitk(a, w, None, a_ready=a_ready, extra_waits=extra_waits, heap_out_off=off + rank * slot_bytes,
                            ld_out=Nn, signal_peer_event=arrived, w_blocked=w_blocked)
        n_arrive = fin.all_event[1]
    else:
        n_arrive = (Nn + bn - 1) // bn

        def per_tile(mb: int, nb: int) -> dict:
            return dict(peer=-2, out_off=off + rank * slot_bytes, signal_peer=-2, signal_peer_event=arrived)

        b.gemm(a, w, slots[0], a_ready=a_ready, extra_waits=extra_waits, bn=bn, per_tile=per_tile)
    row_bytes = Nn * slots.element_size()
    done = b.new_event()
    total = 0
    if reduce_rows is None:
        reduce_rows = max(1, M // b.num_workers)     # latency-bound: spread the rows over the workers
    for r0 in range(0, M, reduce_rows):
        rr = min(reduce_rows, M - r0)
        raw = _pack_comm(off + r0 * row_bytes, 0, row_bytes, row_bytes, row_bytes, rr, N.DTYPE_CODE[slots.dtype], -1,
                         COMM_REDUCE_LOCAL, nslots=world, slot_stride=slot_bytes,
                         local_ptr=out.data_ptr() + r0 * row_bytes,
                         aux_ptr=(residual.data_ptr() + r0 * row_bytes) if residual is not None else 0)
        b.add_task(int(TaskType.ALLREDUCE), raw, waits=[(arrived, world * n_arrive, True, False)], signals=[done])
        total += 1
    b.keepalive += [slots, out] + ([residual] if residual is not None else [])
    return RowEvents(rows=M, block=BM, row_events=[(done, total)], all_event=(done, total))
