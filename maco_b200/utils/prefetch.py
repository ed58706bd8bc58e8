"""Double-buffered host -> device input feed.

``submit(host_tensor)`` starts the copy of the NEXT step's input from pinned host memory on a copy
stream; ``deliver(dst)`` makes the current stream wait for the oldest submitted copy and moves it
into the layer's input buffer with a device-to-device copy (tens of microseconds for tens of MB). A
step that submits the next input right after launching its kernel hides the PCIe transfer behind
the compute, so the end-to-end step time approaches the device time.

The reference offers the building blocks for this (a communication stream and events:
maco/sync/stream_manager.py:41-110) and leaves the pattern to the user.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Optional, Tuple

import torch


class InputPrefetcher:
    def __init__(self, like: torch.Tensor, depth: int = 2, stream: Optional[torch.cuda.Stream] = None):
        if not like.is_cuda:
            raise ValueError("InputPrefetcher stages into CUDA memory")
        self.stream = stream if stream is not None else torch.cuda.Stream(device=like.device)
        self._bufs = [torch.empty_like(like) for _ in range(depth)]
        self._free = [torch.cuda.Event() for _ in range(depth)]
        self._ready = [torch.cuda.Event() for _ in range(depth)]
        self._used = [False] * depth
        self._next = 0
        self._queue: Deque[int] = deque()

    @property
    def pending(self) -> int:
        return len(self._queue)

    def submit(self, host: torch.Tensor) -> None:
        """Starts copying ``host`` (pinned) into the next staging buffer on the copy stream."""
        if len(self._queue) == len(self._bufs):
            raise RuntimeError("every staging buffer holds an undelivered input")
        from ..config import config
        if config.use_pinned_memory and not host.is_pinned():
            # pageable memory would make the copy synchronous with the host: go through a pinned bounce buffer
            if not hasattr(self, "_bounce") or self._bounce.shape != host.shape or self._bounce.dtype != host.dtype:
                self._bounce = [torch.empty(host.shape, dtype=host.dtype).pin_memory() for _ in self._bufs]
            self._bounce[self._next].copy_(host)
            host = self._bounce[self._next]
        i = self._next
        self._next = (i + 1) % len(self._bufs)
        with torch.cuda.stream(self.stream):
            if self._used[i]:
                self.stream.wait_event(self._free[i])       # the previous consumer has read this buffer
            self._bufs[i].copy_(host, non_blocking=True)
            self._ready[i].record(self.stream)
        self._queue.append(i)

    def deliver(self, dst: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """Orders ``stream`` (default: current) behind the oldest submitted copy and moves it into ``dst``."""
        if not self._queue:
            raise RuntimeError("deliver() without a submitted input")
        i = self._queue.popleft()
        cur = stream if stream is not None else torch.cuda.current_stream(dst.device)
        cur.wait_event(self._ready[i])
        with torch.cuda.stream(cur):
            dst.copy_(self._bufs[i], non_blocking=True)
            self._free[i].record(cur)
        self._used[i] = True
        return dst


class StepPipeline:
    """End-to-end step loop with the host one step behind the device.

    ``step(host_input, launch, result)`` does, in stream order: deliver this step's input (its host -> device
    copy was started during the previous step), ``launch()`` the layer, start the copy of the NEXT input,
    copy ``result()`` (a small device tensor) into pinned host memory, and only then wait for the PREVIOUS
    step's result. The host therefore never idles the GPU between steps: the launch of step i+1 is queued
    while step i runs, and the device -> host read of step i completes under step i+1.
    ``drain()`` returns the result of the last step. Every step's input crosses PCIe and every step's result
    is read on the host, each exactly once.

    The reference blocks on the stream after every step (maco/overlap/manager.py:207-208 synchronises both
    events before returning); this keeps the same data movement and removes the bubble.
    """

    def __init__(self, input_buffer, result_like: torch.Tensor, depth: int = 2):
        """``input_buffer``: the layer's input tensor, or a list of TWO alternating input tensors (a layer built
        with two input slots). With two slots the host -> device copy of step i+1 goes straight into the slot that
        step i does not read, and ``launch`` / ``result`` are called with the slot index; with one, inputs are staged
        in side buffers and moved in with a device-to-device copy before each launch."""
        self.slots = list(input_buffer) if isinstance(input_buffer, (list, tuple)) else None
        if self.slots is not None:
            if len(self.slots) != 2:
                raise ValueError("direct input delivery alternates between exactly two input buffers")
            dev = self.slots[0].device
            self._copy_stream = torch.cuda.Stream(device=dev)
            self._ready = [torch.cuda.Event() for _ in range(2)]
            self._free = [torch.cuda.Event() for _ in range(2)]
            self._loaded = [False, False]
            self._consumed = [False, False]
            input_buffer = self.slots[0]
            self.feed = None
        else:
            self.feed = InputPrefetcher(input_buffer, depth=depth)
        self.input_buffer = input_buffer
        from ..config import config
        self._host = [torch.empty(result_like.shape, dtype=result_like.dtype) for _ in range(depth)]
        if config.use_pinned_memory:
            self._host = [h.pin_memory() for h in self._host]
        self._done = [torch.cuda.Event() for _ in range(depth)]
        self._step = 0
        self._pending: Deque[int] = deque()

    def step(self, host_input: torch.Tensor, launch, result, next_host_input: Optional[torch.Tensor] = None):
        """Runs one step; returns the host copy of the previous step's result (None on the first step)."""
        if self.slots is not None:
            return self._step_direct(host_input, launch, result, next_host_input)
        if not self.feed.pending:
            self.feed.submit(host_input)
        self.feed.deliver(self.input_buffer)
        launch()
        self.feed.submit(next_host_input if next_host_input is not None else host_input)
        slot = self._step % len(self._host)
        self._host[slot].copy_(result(), non_blocking=True)
        self._done[slot].record()
        self._pending.append(slot)
        self._step += 1
        if len(self._pending) >= len(self._host):
            return self._pop()
        return None

    def _h2d(self, slot: int, host: torch.Tensor) -> None:
        cs = self._copy_stream
        with torch.cuda.stream(cs):
            if self._consumed[slot]:
                cs.wait_event(self._free[slot])          # the launch that read this slot last has finished
            self.slots[slot].copy_(host, non_blocking=True)
            self._ready[slot].record(cs)
        self._loaded[slot] = True

    def _step_direct(self, host_input, launch, result, next_host_input):
        slot = self._step & 1
        cur = torch.cuda.current_stream(self.slots[0].device)
        if not self._loaded[slot]:
            self._h2d(slot, host_input)
        cur.wait_event(self._ready[slot])
        launch(slot)
        self._free[slot].record(cur)
        self._consumed[slot], self._loaded[slot] = True, False
        self._h2d(slot ^ 1, next_host_input if next_host_input is not None else host_input)
        hs = self._step % len(self._host)
        self._host[hs].copy_(result(slot), non_blocking=True)
        self._done[hs].record()
        self._pending.append(hs)
        self._step += 1
        if len(self._pending) >= len(self._host):
            return self._pop()
        return None

    def _pop(self) -> torch.Tensor:
        slot = self._pending.popleft()
        self._done[slot].synchronize()
        return self._host[slot]

    def drain(self) -> Optional[torch.Tensor]:
        """Waits for every outstanding result; returns the newest."""
        out = None
        while self._pending:
            out = self._pop()
        return out
