"""Per-device compute / communication streams.

API of the reference's StreamManager (maco/sync/stream_manager.py:11-177): one instance per
device, a high-priority compute stream, a communication stream, and event-based cross-stream
waits. Without CUDA the streams are inert stand-ins, so host-side logic (and the CPU tests)
run unchanged.
"""
from __future__ import annotations

import contextlib
from typing import Dict, Optional

import torch


class NullStream:
    """Stand-in for torch.cuda.Stream on a machine without CUDA: work is already synchronous."""

    def synchronize(self) -> None: ...
    def wait_event(self, event) -> None: ...
    def wait_stream(self, stream) -> None: ...
    def record_event(self, event=None):
        return event if event is not None else NullEvent()
    def query(self) -> bool:
        return True


class NullEvent:
    def __init__(self, *a, **k):
        self._recorded = False
    def record(self, stream=None) -> None:
        self._recorded = True
    def wait(self, stream=None) -> None: ...
    def query(self) -> bool:
        return True
    def synchronize(self) -> None: ...
    def elapsed_time(self, other) -> float:
        return 0.0


def has_cuda() -> bool:
    return torch.cuda.is_available()


def new_event(enable_timing: bool = False):
    return torch.cuda.Event(enable_timing=enable_timing) if has_cuda() else NullEvent()


def stream_context(stream):
    if has_cuda() and isinstance(stream, torch.cuda.Stream):
        return torch.cuda.stream(stream)
    return contextlib.nullcontext()


class StreamManager:
    _instances: Dict[int, "StreamManager"] = {}

    def __new__(cls, device: Optional[torch.device] = None):
        idx = cls._device_index(device)
        inst = cls._instances.get(idx)
        if inst is None:
            inst = super().__new__(cls)
            inst._init(idx)
            cls._instances[idx] = inst
        return inst

    @staticmethod
    def _device_index(device) -> int:
        if not has_cuda():
            return -1
        if device is None:
            return torch.cuda.current_device()
        d = torch.device(device)
        return d.index if d.index is not None else torch.cuda.current_device()

    def _init(self, idx: int) -> None:
        self.device_index = idx
        if idx >= 0:
            self.device = torch.device("cuda", idx)
            self._compute_stream = torch.cuda.Stream(device=self.device, priority=-1)
            self._comm_stream = torch.cuda.Stream(device=self.device, priority=0)
        else:
            self.device = torch.device("cpu")
            self._compute_stream = NullStream()
            self._comm_stream = NullStream()

    @property
    def compute_stream(self):
        return self._compute_stream

    @property
    def comm_stream(self):
        return self._comm_stream

    @property
    def default_stream(self):
        return torch.cuda.default_stream(self.device) if self.device_index >= 0 else NullStream()

    def sync_compute(self) -> None:
        self._compute_stream.synchronize()

    def sync_comm(self) -> None:
        self._comm_stream.synchronize()

    def sync_all(self) -> None:
        self._compute_stream.synchronize()
        self._comm_stream.synchronize()

    def _cross_wait(self, waiter, producer) -> None:
        ev = new_event()
        ev.record(producer)
        waiter.wait_event(ev)

    def compute_wait_comm(self) -> None:
        self._cross_wait(self._compute_stream, self._comm_stream)

    def comm_wait_compute(self) -> None:
        self._cross_wait(self._comm_stream, self._compute_stream)

    def default_wait_all(self) -> None:
        d = self.default_stream
        self._cross_wait(d, self._compute_stream)
        self._cross_wait(d, self._comm_stream)

    @classmethod
    def reset(cls) -> None:
        for inst in cls._instances.values():
            try:
                inst.sync_all()
            except Exception:
                pass
        cls._instances.clear()


def get_compute_stream(device=None):
    return StreamManager(device).compute_stream


def get_comm_stream(device=None):
    return StreamManager(device).comm_stream
