"""Signal / wait primitives for ordering work across streams, and their in-kernel counterpart.

API of the reference's maco/sync/signal_wait.py:21-320: ``Signal`` (an event with a name),
``SignalWait`` (named signals plus a wave list), ``OverlapContext`` (compute and comm stream
contexts with the wave numbering compute = 2w, comm = 2w + 1). ``DeviceSignal`` is new: a counter
word in device memory that kernels of this package bump and wait on, so a consumer can start on
the tile a producer just finished instead of on a whole-kernel event.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .stream_manager import NullStream, StreamManager, has_cuda, new_event, stream_context


def _current_stream():
    return torch.cuda.current_stream() if has_cuda() else NullStream()


class Signal:
    def __init__(self, name: str = "", enable_timing: bool = False):
        self.name = name
        self.event = new_event(enable_timing)
        self.signaled = False
        self.stream = None

    def record(self, stream=None) -> "Signal":
        s = stream if stream is not None else _current_stream()
        self.event.record(s) if has_cuda() else self.event.record()
        self.signaled = True
        self.stream = s
        return self

    def wait(self, stream=None) -> None:
        """Makes ``stream`` (default: the current stream) wait for the signal; the host does not block."""
        if not self.signaled:
            return
        s = stream if stream is not None else _current_stream()
        s.wait_event(self.event)

    def is_ready(self) -> bool:
        return self.signaled and self.event.query()

    def synchronize(self) -> None:
        if self.signaled:
            self.event.synchronize()


def create_signal(name: str = "", enable_timing: bool = False) -> Signal:
    return Signal(name, enable_timing)


class SignalWait:
    def __init__(self):
        self._signals: Dict[str, Signal] = {}
        self._waves: List[Optional[Signal]] = []

    def create_signal(self, name: str) -> Signal:
        sig = Signal(name)
        self._signals[name] = sig
        return sig

    def get_signal(self, name: str) -> Optional[Signal]:
        return self._signals.get(name)

    def signal(self, name: str, stream=None) -> Signal:
        sig = self._signals.get(name) or self.create_signal(name)
        return sig.record(stream)

    def wait(self, name: str, stream=None) -> None:
        sig = self._signals.get(name)
        if sig is None:
            raise KeyError(f"no signal named {name!r}")
        sig.wait(stream)

    def signal_wave(self, wave_id: int, stream=None) -> Signal:
        while len(self._waves) <= wave_id:
            self._waves.append(None)
        sig = Signal(f"wave_{wave_id}")
        self._waves[wave_id] = sig
        return sig.record(stream)

    def wait_wave(self, wave_id: int, stream=None) -> None:
        if 0 <= wave_id < len(self._waves) and self._waves[wave_id] is not None:
            self._waves[wave_id].wait(stream)

    def wait_all_waves(self, stream=None) -> None:
        for sig in self._waves:
            if sig is not None:
                sig.wait(stream)

    def synchronize(self) -> None:
        for sig in list(self._signals.values()) + [w for w in self._waves if w is not None]:
            sig.synchronize()

    def reset(self) -> None:
        self._signals.clear()
        self._waves.clear()

    @property
    def num_waves(self) -> int:
        return len(self._waves)


class OverlapContext:
    """Two stream contexts and per-wave signals: compute of wave w records signal 2w, comm of
    wave w records 2w + 1."""

    def __init__(self, device=None):
        self._sm = StreamManager(device)
        self._sw = SignalWait()

    @property
    def compute_stream(self):
        return self._sm.compute_stream

    @property
    def comm_stream(self):
        return self._sm.comm_stream

    @property
    def signals(self) -> SignalWait:
        return self._sw

    def compute(self):
        return stream_context(self._sm.compute_stream)

    def comm(self):
        return stream_context(self._sm.comm_stream)

    def signal_compute_done(self, wave_id: int = 0) -> None:
        self._sw.signal_wave(2 * wave_id, self._sm.compute_stream)

    def signal_comm_done(self, wave_id: int = 0) -> None:
        self._sw.signal_wave(2 * wave_id + 1, self._sm.comm_stream)

    def wait_compute_done(self, wave_id: int = 0) -> None:
        self._sw.wait_wave(2 * wave_id, self._sm.comm_stream)

    def wait_comm_done(self, wave_id: int = 0) -> None:
        self._sw.wait_wave(2 * wave_id + 1, self._sm.compute_stream)

    def sync_all(self) -> None:
        self._sm.sync_all()

    def reset(self) -> None:
        self._sw.reset()


class DeviceSignal:
    """A monotonically increasing 32-bit counter in device memory used as a signal by kernels.

    ``tensor`` is a 1-element int32 CUDA tensor (inside the symmetric heap when peers must see
    it). ``Program.event_signal(e)`` hands out the counters of a persistent-kernel program's events in this
    form: tasks add to them with release semantics and wait on them with acquire semantics and a time
    budget; the host can read them, or wait on them with a bound, while a launch is running.
    """

    def __init__(self, tensor: Optional[torch.Tensor] = None, device=None):
        if tensor is None:
            tensor = torch.zeros(1, dtype=torch.int32, device=device or ("cuda" if has_cuda() else "cpu"))
        if tensor.dtype != torch.int32 or tensor.numel() != 1:
            raise ValueError("DeviceSignal needs a 1-element int32 tensor")
        self.tensor = tensor

    @property
    def ptr(self) -> int:
        return self.tensor.data_ptr()

    def value(self) -> int:
        return int(self.tensor.item())

    def reset(self) -> None:
        self.tensor.zero_()

    def wait_value(self, value: int, timeout_s: float = 10.0, poll_s: float = 1e-4) -> bool:
        """Host-side bounded wait until the counter reaches ``value`` (wrap-safe). Reads go through a side stream,
        so a kernel that is still running on the current stream does not block them. Returns False on timeout."""
        import time
        if not self.tensor.is_cuda:
            return ((int(self.tensor.item()) - value) & 0xFFFFFFFF) < 0x80000000
        if not hasattr(self, "_side"):
            self._side = torch.cuda.Stream(device=self.tensor.device)
            self._host = torch.zeros(1, dtype=torch.int32).pin_memory()
        t0 = time.monotonic()
        while True:
            with torch.cuda.stream(self._side):
                self._host.copy_(self.tensor, non_blocking=True)
            self._side.synchronize()
            if ((int(self._host.item()) - value) & 0xFFFFFFFF) < 0x80000000:
                return True
            if time.monotonic() - t0 > timeout_s:
                return False
            time.sleep(poll_s)
