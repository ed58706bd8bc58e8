"""Stand-alone collectives served by the persistent kernel's communication tasks.

Each call builds (once, then caches) a small program over a buffer of the symmetric heap and
launches it: all ranks' kernels pull / push over NVLink peer memory and synchronise through
event counters in the heap. These back ``comm.patterns`` when ``config.backend == "peer"``, and
the ``nvshmem_*`` compatibility calls. NCCL stays available as the baseline (``comm.nccl_ops``).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .. import _native as N
from ..ops.megakernel import COMM_PUSH, Program, ProgramBuilder, _pack_comm
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
        b = _builder(heap, workers=max(1, min(32, (t.numel() * t.element_size()) >> 18)))
        fence = fused.epoch_fence_event(b)
        ready = b.new_event()
        b.add_task(int(TaskType.NOP), b"", waits=[fence], signal_peer=-2, signal_peer_event=ready)
        flat = t.view(-1)
        done, n = fused.allreduce_tasks(b, flat, avg=avg, chunk_bytes=256 << 10, ready_event=ready, comm_worker=False)
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


def clear_cache() -> None:
    _cache.clear()
    _scratch.clear()
