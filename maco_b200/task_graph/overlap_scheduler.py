"""Wave-overlap planner and two-stream executor.

API of the reference's maco/task_graph/overlap_scheduler.py:19-296 (``OverlapMode``,
``OverlapPlan``, ``OverlapScheduler.create_plan / execute_plan``, ``OverlapRuntime``).

Executor differences: the reference makes wave w+1's compute wait for wave w's *communication*
(overlap_scheduler.py:191-231), so at most one compute and one comm wave are ever in flight.
Here compute waves are only ordered among themselves; communication of wave w waits for compute
of wave w and for communication of wave w-1, so the comm stream can trail the compute stream by
any number of waves. ``PIPELINE`` mode (an enum value without an implementation in the
reference) issues all compute first-come on the compute stream and each wave's communication as
soon as its compute event fires, without any back edge.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional

import torch

from ..sync.signal_wait import SignalWait
from ..sync.stream_manager import StreamManager, stream_context


class OverlapMode(Enum):
    NONE = "none"
    WAVE = "wave"
    PIPELINE = "pipeline"


@dataclass
class OverlapPlan:
    mode: OverlapMode
    num_waves: int
    compute_waves: List[list] = field(default_factory=list)
    comm_tasks: list = field(default_factory=list)
    wave_comm_mapping: Dict[int, list] = field(default_factory=dict)


class OverlapScheduler:
    def __init__(self, device: Optional[torch.device] = None):
        self.stream_manager = StreamManager(device)
        self.signals = SignalWait()

    def create_plan(self, compute_tasks: list, comm_tasks: list, mode: OverlapMode = OverlapMode.WAVE,
                    num_waves: Optional[int] = None) -> OverlapPlan:
        compute_tasks, comm_tasks = list(compute_tasks), list(comm_tasks)
        if mode == OverlapMode.NONE or not comm_tasks or not compute_tasks:
            return OverlapPlan(mode=OverlapMode.NONE if mode == OverlapMode.NONE else mode, num_waves=1,
                               compute_waves=[compute_tasks], comm_tasks=comm_tasks,
                               wave_comm_mapping={0: comm_tasks})
        if num_waves is None:
            num_waves = self._auto_determine_waves(compute_tasks, comm_tasks)
        num_waves = max(1, min(int(num_waves), len(compute_tasks)))
        waves = self._partition_waves(compute_tasks, num_waves)
        mapping = self._map_waves_to_comm(len(waves), comm_tasks)
        return OverlapPlan(mode=mode, num_waves=len(waves), compute_waves=waves, comm_tasks=comm_tasks,
                           wave_comm_mapping=mapping)

    @staticmethod
    def _auto_determine_waves(compute_tasks: list, comm_tasks: list) -> int:
        return max(1, min(len(comm_tasks), len(compute_tasks) // 2))

    @staticmethod
    def _partition_waves(tasks: list, num_waves: int) -> List[list]:
        n = len(tasks)
        base, extra = divmod(n, num_waves)
        waves, pos = [], 0
        for w in range(num_waves):
            size = base + (1 if w < extra else 0)
            if size:
                waves.append(tasks[pos:pos + size])
            pos += size
        return waves

    @staticmethod
    def _map_waves_to_comm(num_waves: int, comm_tasks: list) -> Dict[int, list]:
        mapping: Dict[int, list] = {w: [] for w in range(num_waves)}
        for i, t in enumerate(comm_tasks):
            mapping[i % num_waves].append(t)
        return mapping

    def execute_plan(self, plan: OverlapPlan, compute_fn: Callable, comm_fn: Callable) -> None:
        if plan.mode == OverlapMode.NONE:
            for wave in plan.compute_waves:
                for t in wave:
                    compute_fn(t)
            for t in plan.comm_tasks:
                comm_fn(t)
            return
        self._execute_wave_overlap(plan, compute_fn, comm_fn)

    def _execute_wave_overlap(self, plan: OverlapPlan, compute_fn: Callable, comm_fn: Callable) -> None:
        sm, sw = self.stream_manager, self.signals
        sw.reset()
        cs, ms = sm.compute_stream, sm.comm_stream
        if hasattr(cs, "wait_stream") and torch.cuda.is_available():
            cur = torch.cuda.current_stream()
            cs.wait_stream(cur)
            ms.wait_stream(cur)
        for w, tasks in enumerate(plan.compute_waves):
            with stream_context(cs):
                for t in tasks:
                    compute_fn(t)
            sw.signal_wave(2 * w, cs)
            comm = plan.wave_comm_mapping.get(w, [])
            if comm:
                sw.wait_wave(2 * w, ms)
                with stream_context(ms):
                    for t in comm:
                        comm_fn(t)
            sw.signal_wave(2 * w + 1, ms)
        sm.sync_all()


class OverlapRuntime:
    def __init__(self, device: Optional[torch.device] = None):
        self.scheduler = OverlapScheduler(device)

    def execute_overlap(self, compute_tasks: list, comm_tasks: list, compute_executor: Callable,
                        comm_executor: Callable, mode: Optional[OverlapMode] = None,
                        num_waves: Optional[int] = None) -> None:
        """``mode`` None takes ``config.overlap_strategy``: "auto" / "wave" -> WAVE, "pipeline" -> PIPELINE,
        "none" -> NONE (compute, then communication, on one stream)."""
        if mode is None:
            from ..config import config
            mode = {"none": OverlapMode.NONE, "pipeline": OverlapMode.PIPELINE}.get(str(config.overlap_strategy).lower(),
                                                                                    OverlapMode.WAVE)
        plan = self.scheduler.create_plan(compute_tasks, comm_tasks, mode=mode, num_waves=num_waves)
        self.scheduler.execute_plan(plan, compute_executor, comm_executor)

    @property
    def compute_stream(self):
        return self.scheduler.stream_manager.compute_stream

    @property
    def comm_stream(self):
        return self.scheduler.stream_manager.comm_stream
