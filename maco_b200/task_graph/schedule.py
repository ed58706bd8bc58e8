"""Topological schedule of a task graph: execution waves and worker assignment.

Counterpart of TaskSchedule in the reference (maco/task_graph/__init__.py:209-269). Waves are
Kahn levels computed in O(nodes + edges) (the reference rebuilds id lists inside a nested loop,
O(waves * n^2)).
"""
from __future__ import annotations

from typing import Dict, List

from .nodes import TaskNode


class TaskSchedule:
    def __init__(self, nodes: List[TaskNode], num_workers: int):
        self.nodes = list(nodes)
        self.num_workers = max(1, int(num_workers))
        self.waves: List[List[TaskNode]] = []
        self.worker_assignments: Dict[int, int] = {}
        self.order: List[TaskNode] = []
        self._compute_waves()
        self._assign_workers()

    def _compute_waves(self) -> None:
        indeg = {id(n): 0 for n in self.nodes}
        users: Dict[int, List[TaskNode]] = {id(n): [] for n in self.nodes}
        for n in self.nodes:
            for d in n.depends_on:
                if id(d) in indeg:
                    indeg[id(n)] += 1
                    users[id(d)].append(n)
        frontier = [n for n in self.nodes if indeg[id(n)] == 0]
        while frontier:
            frontier.sort(key=lambda t: (-t.priority, t._node_id))
            self.waves.append(frontier)
            self.order.extend(frontier)
            nxt: List[TaskNode] = []
            for n in frontier:
                for u in users[id(n)]:
                    indeg[id(u)] -= 1
                    if indeg[id(u)] == 0:
                        nxt.append(u)
            frontier = nxt

    def _assign_workers(self) -> None:
        rr = 0
        for wave in self.waves:
            for n in wave:
                if n.target_worker is not None:
                    self.worker_assignments[n._node_id] = int(n.target_worker) % self.num_workers
                else:
                    self.worker_assignments[n._node_id] = rr % self.num_workers
                    rr += 1

    def __len__(self) -> int:
        return len(self.nodes)
