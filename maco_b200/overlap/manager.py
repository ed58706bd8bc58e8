"""Two-stream compute / communication overlap manager.

API of the reference's OverlapManager / OverlapRegion (maco/overlap/manager.py:15-434): run a
compute callable on the compute stream while a collective (or any communication callable) runs
on the comm stream, with events fencing both against the caller's stream. On CPU (no CUDA) the
two run back to back. The ``stats`` dict is filled (the reference never updates it).
"""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..sync.stream_manager import NullStream, has_cuda, new_event, stream_context


@dataclass
class OverlapTask:
    fn: Callable
    args: tuple = ()
    kwargs: dict = None
    event: Any = None
    result: Any = None


class _FutureResult:
    def __init__(self, event, result):
        self._event = event
        self._result = result

    def wait(self):
        if self._event is not None:
            self._event.synchronize()
        return self._result

    def result(self):
        return self.wait()


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _run_collective(tensor: torch.Tensor, op: str, **kwargs):
    from ..comm import patterns
    if op == "allreduce":
        return patterns.allreduce(tensor, op=kwargs.get("reduce_op", "sum"))
    if op == "allgather":
        return patterns.allgather(tensor)
    if op == "reduce_scatter":
        return patterns.reduce_scatter(tensor, op=kwargs.get("reduce_op", "sum"))
    if op == "all_to_all":
        return patterns.all_to_all(tensor, kwargs.get("scatter_dim", 0), kwargs.get("gather_dim", 0))
    if op == "broadcast":
        if _world() > 1:
            dist.broadcast(tensor, src=kwargs.get("src", 0))
        return tensor
    raise ValueError(f"unknown communication op {op!r}")


class OverlapManager:
    def __init__(self, device: Optional[torch.device] = None):
        self.cuda = has_cuda() and (device is None or torch.device(device).type == "cuda")
        if self.cuda:
            self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
            self.compute_stream = torch.cuda.Stream(device=self.device, priority=-1)
            self.comm_stream = torch.cuda.Stream(device=self.device)
        else:
            self.device = torch.device("cpu")
            self.compute_stream = None
            self.comm_stream = None
        self.stats = {"num_overlaps": 0, "compute_tasks": 0, "comm_tasks": 0, "sync_calls": 0}

    def get_comm_stream(self):
        return self.comm_stream

    def get_compute_stream(self):
        return self.compute_stream

    def sync_streams(self) -> None:
        self.stats["sync_calls"] += 1
        if self.cuda:
            self.compute_stream.synchronize()
            self.comm_stream.synchronize()

    synchronize = sync_streams

    @contextmanager
    def overlap_region(self):
        region = OverlapRegion(self)
        try:
            yield region
        finally:
            region.wait_all()

    def _fork(self, stream) -> None:
        stream.wait_stream(torch.cuda.current_stream(self.device))

    def submit_compute(self, fn: Callable, *args, **kwargs):
        self.stats["compute_tasks"] += 1
        if not self.cuda:
            return None, fn(*args, **kwargs)
        self._fork(self.compute_stream)
        ev = torch.cuda.Event()
        with torch.cuda.stream(self.compute_stream):
            result = fn(*args, **kwargs)
            ev.record()
        return ev, result

    def submit_comm(self, tensor: torch.Tensor, op: str = "allreduce", **kwargs):
        self.stats["comm_tasks"] += 1
        if not self.cuda or not tensor.is_cuda:
            return None, _run_collective(tensor, op, **kwargs)
        self._fork(self.comm_stream)
        ev = torch.cuda.Event()
        with torch.cuda.stream(self.comm_stream):
            result = _run_collective(tensor, op, **kwargs)
            ev.record()
        tensor.record_stream(self.comm_stream)
        return ev, result

    def overlap_compute_and_comm(self, compute_fn: Callable[[], Any], comm_tensor: torch.Tensor,
                                 comm_op: str = "allreduce", **kwargs) -> Tuple[Any, Any]:
        """Returns ``(compute_result, comm_result)``; both are complete with respect to the current stream."""
        self.stats["num_overlaps"] += 1
        cev, comm_result = self.submit_comm(comm_tensor, comm_op, **kwargs)
        pev, compute_result = self.submit_compute(compute_fn)
        self._join(cev, pev)
        return compute_result, comm_result

    def overlap_all_to_all_with_compute(self, all_to_all_fn: Callable[[], Any], compute_fn: Callable[[], Any]):
        """Returns ``(all_to_all_result, compute_result)``."""
        return self.overlap_generic(all_to_all_fn, compute_fn)

    def overlap_generic(self, comm_fn: Callable[[], Any], compute_fn: Callable[[], Any]):
        self.stats["num_overlaps"] += 1
        if not self.cuda:
            return comm_fn(), compute_fn()
        self._fork(self.comm_stream)
        cev = torch.cuda.Event()
        with torch.cuda.stream(self.comm_stream):
            comm_result = comm_fn()
            cev.record()
        pev, compute_result = self.submit_compute(compute_fn)
        self._join(cev, pev)
        return comm_result, compute_result

    def _join(self, *events) -> None:
        if not self.cuda:
            return
        cur = torch.cuda.current_stream(self.device)
        for ev in events:
            if ev is not None:
                cur.wait_event(ev)


class OverlapRegion:
    """Collects communication and compute callables issued inside ``with manager.overlap_region()``."""

    def __init__(self, manager: OverlapManager):
        self.manager = manager
        self._comm: List[_FutureResult] = []
        self._compute: List[_FutureResult] = []
        self._events: List[Any] = []

    def comm(self, fn: Callable) -> _FutureResult:
        m = self.manager
        if not m.cuda:
            fut = _FutureResult(None, fn())
        else:
            m._fork(m.comm_stream)
            ev = torch.cuda.Event()
            with torch.cuda.stream(m.comm_stream):
                res = fn()
                ev.record()
            self._events.append(ev)
            fut = _FutureResult(ev, res)
        self._comm.append(fut)
        return fut

    def compute(self, fn: Callable) -> _FutureResult:
        m = self.manager
        ev, res = m.submit_compute(fn)
        if ev is not None:
            self._events.append(ev)
        fut = _FutureResult(ev, res)
        self._compute.append(fut)
        return fut

    def submit_compute(self, fn: Callable, *args, **kwargs) -> _FutureResult:
        return self.compute(lambda: fn(*args, **kwargs))

    def submit_comm(self, tensor: torch.Tensor, op: str = "allreduce", **kwargs) -> _FutureResult:
        return self.comm(lambda: _run_collective(tensor, op, **kwargs))

    def get_comm_results(self) -> List[Any]:
        return [f.result() for f in self._comm]

    def get_compute_results(self) -> List[Any]:
        return [f.result() for f in self._compute]

    def wait_all(self) -> None:
        self.manager._join(*self._events)
        self._events.clear()
