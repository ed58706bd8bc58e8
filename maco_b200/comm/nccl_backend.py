"""Library-collective backend with two-stream overlap (the NCCL baseline backend).

API of the reference's NCCLBackend (maco/comm/nccl_backend.py:17-350): ``OverlapMode``,
``CommHandle``, ``allreduce`` / ``allreduce_overlap`` / ``allgather`` / ``reduce_scatter`` /
``barrier`` / ``synchronize_streams``, the ``stats`` dict and the ``get_backend`` / ``init_backend``
globals. Two fixes: the streams exist as soon as CUDA does (the reference creates them only in
an ``init_process_group`` call that ``maco.init`` never makes, so its global backend never
overlaps), and the stats are filled from CUDA-event timings.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


class OverlapMode(Enum):
    NONE = "none"
    STREAM = "stream"
    PERSISTENT = "persistent"


@dataclass
class CommHandle:
    tensor: torch.Tensor
    work: Optional[Any] = None
    stream: Optional[Any] = None
    event: Optional[Any] = None
    completed: bool = False

    def wait(self) -> torch.Tensor:
        if not self.completed:
            if self.work is not None:
                self.work.wait()
            if self.event is not None:
                torch.cuda.current_stream().wait_event(self.event)
            self.completed = True
        return self.tensor

    def is_completed(self) -> bool:
        if self.completed:
            return True
        if self.event is not None:
            return self.event.query()
        if self.work is not None:
            return self.work.is_completed()
        return True


class NCCLBackend:
    def __init__(self, rank: int = 0, world_size: int = 1, overlap_mode: OverlapMode = OverlapMode.STREAM):
        self.rank = rank
        self.world_size = world_size
        self.overlap_mode = overlap_mode
        self._initialized = False
        self.compute_stream = None
        self.comm_stream = None
        self.stats = {"allreduce_count": 0, "allreduce_time_ms": 0.0, "overlap_time_saved_ms": 0.0}
        self._timed: List[Tuple[Any, Any]] = []
        self._ensure_streams()

    def _ensure_streams(self) -> None:
        if self.overlap_mode != OverlapMode.NONE and torch.cuda.is_available() and self.comm_stream is None:
            self.compute_stream = torch.cuda.Stream(priority=-1)
            self.comm_stream = torch.cuda.Stream()

    def init_process_group(self, backend: str = "nccl", init_method: str = "env://") -> None:
        if self._initialized:
            return
        if not dist.is_initialized() and self.world_size > 1:
            dist.init_process_group(backend=backend, init_method=init_method, rank=self.rank, world_size=self.world_size)
        if dist.is_initialized():
            self.rank, self.world_size = dist.get_rank(), dist.get_world_size()
        self._ensure_streams()
        self._initialized = True

    def _multi(self) -> bool:
        return self.world_size > 1 and dist.is_initialized()

    def allreduce(self, tensor: torch.Tensor, op=None, async_op: bool = False) -> CommHandle:
        op = op if op is not None else dist.ReduceOp.SUM
        self.stats["allreduce_count"] += 1
        if not self._multi():
            return CommHandle(tensor=tensor, completed=True)
        if tensor.is_cuda and self.comm_stream is not None:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                start.record()
                dist.all_reduce(tensor, op=op)
                end.record()
            tensor.record_stream(self.comm_stream)
            self._timed.append((start, end))
            h = CommHandle(tensor=tensor, stream=self.comm_stream, event=end)
            if not async_op:
                h.wait()
            return h
        work = dist.all_reduce(tensor, op=op, async_op=async_op)
        return CommHandle(tensor=tensor, work=work if async_op else None, completed=not async_op)

    def allreduce_overlap(self, tensor: torch.Tensor, compute_fn: Callable[[], Any], op=None):
        """Runs ``compute_fn`` on the compute stream while ``tensor`` is all-reduced on the comm stream."""
        h = self.allreduce(tensor, op=op, async_op=True)
        if tensor.is_cuda and self.compute_stream is not None:
            cur = torch.cuda.current_stream()
            self.compute_stream.wait_stream(cur)
            with torch.cuda.stream(self.compute_stream):
                result = compute_fn()
            cur.wait_stream(self.compute_stream)
        else:
            result = compute_fn()
        h.wait()
        return tensor, result

    def allgather(self, tensor: torch.Tensor, async_op: bool = False):
        if not self._multi():
            return tensor.unsqueeze(0)
        out = torch.empty((self.world_size,) + tuple(tensor.shape), dtype=tensor.dtype, device=tensor.device)
        dist.all_gather_into_tensor(out.view(-1, *tensor.shape[1:]) if tensor.dim() else out, tensor.contiguous())
        return out

    def reduce_scatter(self, tensor: torch.Tensor, op=None):
        from . import patterns
        if not self._multi():
            return tensor
        return patterns.reduce_scatter(tensor, op=op if op is not None else patterns.ReduceOp.SUM)

    def barrier(self) -> None:
        if self._multi():
            dist.barrier()

    def synchronize_streams(self) -> None:
        for s in (self.compute_stream, self.comm_stream):
            if s is not None:
                s.synchronize()
        self._drain_timings()

    def _drain_timings(self) -> None:
        left = []
        for s, e in self._timed:
            if e.query():
                self.stats["allreduce_time_ms"] += s.elapsed_time(e)
            else:
                left.append((s, e))
        self._timed = left

    def get_stats(self) -> dict:
        self._drain_timings()
        return dict(self.stats)

    def cleanup(self) -> None:
        self.synchronize_streams()
        self._initialized = False


_backend: Optional[NCCLBackend] = None


def get_backend() -> Optional[NCCLBackend]:
    return _backend


def init_backend(rank: int = 0, world_size: int = 1, overlap_mode: OverlapMode = OverlapMode.STREAM) -> NCCLBackend:
    global _backend
    _backend = NCCLBackend(rank=rank, world_size=world_size, overlap_mode=overlap_mode)
    _backend._initialized = True
    return _backend
