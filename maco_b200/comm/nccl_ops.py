"""Asynchronous collectives on a side stream, through torch.distributed (NCCL or gloo).

API of the reference's maco/comm/nccl_ops.py:16-356 (``AsyncHandle`` and the ``async_*`` calls).
This is the library-collective path: the baseline the in-kernel peer-memory collectives are
measured against, and the path CPU (gloo) ranks use. With a world size of 1 every call is the
identity.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ._compat import list_all_to_all
from .process_group import get_world_size

_comm_streams = {}


def _use_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


def _get_comm_stream(device=None):
    if not torch.cuda.is_available():
        return None
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _comm_streams:
        _comm_streams[idx] = torch.cuda.Stream(device=idx)
    return _comm_streams[idx]


class AsyncHandle:
    """Completion handle of an asynchronous collective."""

    def __init__(self, work=None, stream=None, event=None, output=None, finalize=None):
        self.work = work
        self.stream = stream
        self.event = event
        self.output = output
        self._finalize = finalize
        self._done = False

    def wait(self):
        if not self._done:
            if self.work is not None:
                self.work.wait()
            if self.event is not None:
                torch.cuda.current_stream().wait_event(self.event)
            if self._finalize is not None:
                self.output = self._finalize()
            self._done = True
        return self.output

    def is_completed(self) -> bool:
        if self._done:
            return True
        if self.event is not None:
            return self.event.query()
        if self.work is not None:
            return self.work.is_completed()
        return True


def _launch(t: torch.Tensor, fn, async_op: bool, output=None, finalize=None) -> AsyncHandle:
    """Runs ``fn()`` (which issues the collective) on the comm stream after the current stream."""
    if _use_cuda(t):
        stream = _get_comm_stream(t.device)
        stream.wait_stream(torch.cuda.current_stream(t.device))
        with torch.cuda.stream(stream):
            work = fn()
            ev = torch.cuda.Event()
            ev.record(stream)
        h = AsyncHandle(work=None, stream=stream, event=ev, output=output, finalize=finalize)
        for x in ([t] + ([output] if isinstance(output, torch.Tensor) else [])):
            x.record_stream(stream)
    else:
        work = fn()
        h = AsyncHandle(work=work if async_op else None, output=output, finalize=finalize)
        if not async_op and work is not None and hasattr(work, "wait"):
            work.wait()
    if not async_op:
        h.wait()
    return h


def async_all_reduce(tensor: torch.Tensor, op=None, group=None, async_op: bool = True) -> AsyncHandle:
    op = op if op is not None else dist.ReduceOp.SUM
    if get_world_size() == 1:
        return AsyncHandle(output=tensor)
    return _launch(tensor, lambda: dist.all_reduce(tensor, op=op, group=group, async_op=True), async_op, output=tensor)


def async_all_gather(tensor: torch.Tensor, group=None, async_op: bool = True) -> AsyncHandle:
    """Gathers along dim 0: result is ``[world * n, ...]``."""
    world = get_world_size()
    if world == 1:
        return AsyncHandle(output=tensor)
    out = torch.empty((world * tensor.shape[0],) + tuple(tensor.shape[1:]), dtype=tensor.dtype, device=tensor.device)
    src = tensor.contiguous()
    return _launch(tensor, lambda: dist.all_gather_into_tensor(out, src, group=group, async_op=True), async_op, output=out)


def async_all_to_all(tensor: torch.Tensor, scatter_dim: int = 0, gather_dim: int = 0, group=None,
                     async_op: bool = True) -> AsyncHandle:
    """Splits ``scatter_dim`` over ranks, concatenates received pieces along ``gather_dim``."""
    world = get_world_size()
    if world == 1:
        return AsyncHandle(output=tensor)
    send = [c.contiguous() for c in tensor.chunk(world, dim=scatter_dim)]
    recv = [torch.empty_like(send[0]) for _ in range(world)]
    return _launch(tensor, lambda: list_all_to_all(recv, send, group=group, async_op=True), async_op,
                   output=None, finalize=lambda: torch.cat(recv, dim=gather_dim))


def async_all_to_all_4d(tensor: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1, group=None,
                        async_op: bool = True) -> AsyncHandle:
    if tensor.dim() != 4:
        raise ValueError(f"async_all_to_all_4d expects a 4-D tensor, got {tensor.dim()}-D")
    return async_all_to_all(tensor, scatter_dim=scatter_dim, gather_dim=gather_dim, group=group, async_op=async_op)


def async_broadcast(tensor: torch.Tensor, src: int = 0, group=None, async_op: bool = True) -> AsyncHandle:
    if get_world_size() == 1:
        return AsyncHandle(output=tensor)
    return _launch(tensor, lambda: dist.broadcast(tensor, src=src, group=group, async_op=True), async_op, output=tensor)


def sync_stream() -> None:
    s = _get_comm_stream()
    if s is not None:
        s.synchronize()


def wait_comm_stream() -> None:
    """Makes the current stream wait for everything queued on the comm stream."""
    s = _get_comm_stream()
    if s is not None:
        torch.cuda.current_stream().wait_stream(s)
