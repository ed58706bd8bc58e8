"""Node types of the task graph: TaskType, TaskNode, OverlapGroup.

API parity with the reference's maco/task_graph/__init__.py:65-206. The numeric TaskType values are
the ones the native task kernel uses too (csrc/maco_types.h), which the reference's two enums do
not manage (its Python LINEAR=101 is its C ATTENTION).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import IntEnum
from typing import Any, Callable, Dict, List, Optional

import torch


class TaskType(IntEnum):
    TERMINATE = 0
    NOP = 1
    # compute: 100 <= v < 200
    MATMUL = 100
    LINEAR = 101
    ATTENTION = 102
    LAYERNORM = 103
    RMSNORM = 104
    GELU = 105
    SILU = 106
    SOFTMAX = 107
    SILU_GATE = 108
    ROPE = 109
    TOPK = 110
    ATTN_MERGE = 111
    SCALE = 112
    ADD = 113
    GELU_BWD = 114
    AXPBY = 115
    CUSTOM_COMPUTE = 150
    # communication: 200 <= v < 300
    ALLREDUCE = 200
    ALLGATHER = 201
    REDUCE_SCATTER = 202
    ALL_TO_ALL = 203
    BROADCAST = 204
    PEER_BARRIER = 205
    CUSTOM_COMM = 250
    # memory
    COPY = 300


@dataclass(eq=False)
class TaskNode:
    """One operation of the graph. ``outputs`` are allocated when the node is created."""

    name: str
    task_type: TaskType
    inputs: List[torch.Tensor] = field(default_factory=list)
    outputs: List[torch.Tensor] = field(default_factory=list)
    dims: List[int] = field(default_factory=list)
    depends_on: List["TaskNode"] = field(default_factory=list)
    priority: int = 0
    target_worker: Optional[int] = None
    custom_fn: Optional[Callable] = None
    attrs: Dict[str, Any] = field(default_factory=dict)
    _node_id: int = -1
    _event_id: int = -1
    _wave_id: int = 0
    _overlap_role: Optional[str] = None
    _overlap_group: Optional["OverlapGroup"] = field(default=None, repr=False)

    def add_dependency(self, *tasks: "TaskNode") -> "TaskNode":
        for t in tasks:
            if t is not None and t is not self and t not in self.depends_on:
                self.depends_on.append(t)
        return self

    @property
    def output(self) -> Optional[torch.Tensor]:
        return self.outputs[0] if self.outputs else None

    @property
    def is_compute(self) -> bool:
        return 100 <= int(self.task_type) < 200

    @property
    def is_comm(self) -> bool:
        return 200 <= int(self.task_type) < 300

    def __repr__(self) -> str:
        return f"TaskNode({self.name!r}, {self.task_type.name}, id={self._node_id})"

    def __hash__(self) -> int:
        return id(self)


class OverlapGroup:
    """Marks compute tasks and communication tasks that should run concurrently.

    The compute tasks are split into ``num_waves`` contiguous waves; communication task ``j`` is
    attached to wave ``j % num_waves`` and may start as soon as that wave's compute has finished,
    while later waves keep computing. Unlike the reference, where the wave ids are written and
    never read (maco/task_graph/runtime.py:160-171), both runtimes here act on them: the stream
    runtime puts the group's communication on the comm stream behind a per-wave event, the
    persistent runtime routes it to the communication workers.
    """

    def __init__(self, graph, compute_tasks: List[TaskNode], comm_tasks: List[TaskNode]):
        self.graph = graph
        self.compute_tasks = list(compute_tasks)
        self.comm_tasks = list(comm_tasks)
        self.num_waves = 1
        self._explicit = False
        for t in self.compute_tasks:
            t._overlap_role = "compute"
            t._overlap_group = self
        for t in self.comm_tasks:
            t._overlap_role = "comm"
            t._overlap_group = self

    def with_waves(self, num_waves: int) -> "OverlapGroup":
        if num_waves < 1:
            raise ValueError("num_waves must be >= 1")
        self.num_waves = int(num_waves)
        self._explicit = True
        self._assign_waves()
        return self

    def auto_waves(self) -> "OverlapGroup":
        n = len(self.compute_tasks)
        self.num_waves = 1 if n <= 2 else (2 if n <= 8 else 4)
        self._explicit = True
        self._assign_waves()
        return self

    def _assign_waves(self) -> None:
        n = len(self.compute_tasks)
        per_wave = max(1, n // self.num_waves)
        for i, t in enumerate(self.compute_tasks):
            t._wave_id = min(i // per_wave, self.num_waves - 1)
        for j, t in enumerate(self.comm_tasks):
            t._wave_id = j % self.num_waves

    def wave(self, w: int) -> List[TaskNode]:
        return [t for t in self.compute_tasks if t._wave_id == w]
