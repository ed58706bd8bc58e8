"""Phase-based communication scheduler: named phases of collectives with dependencies.

API of the reference's CommScheduler (maco/comm/scheduler.py:13-267): build phases with
``phase(name, depends_on=[...]).allreduce(t).allgather(t)...``, ``compile()`` orders them
topologically (raising on a cycle), ``execute()`` runs them through :mod:`patterns`.
``num_sms`` is no longer decorative: it is handed to the peer-memory collectives as their CTA
budget, so a phase can be kept off the SMs a concurrent GEMM needs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional

import torch

from . import patterns


class CommOpType(Enum):
    ALLREDUCE = "allreduce"
    ALLGATHER = "allgather"
    REDUCE_SCATTER = "reduce_scatter"
    SEND = "send"
    RECV = "recv"
    ALL_TO_ALL = "all_to_all"
    BROADCAST = "broadcast"


@dataclass
class CommOp:
    op_type: CommOpType
    tensor: torch.Tensor
    kwargs: Dict[str, Any] = field(default_factory=dict)
    handle: Any = None
    result: Any = None


class CommPhase:
    def __init__(self, name: str, depends_on: Optional[List[str]] = None):
        self.name = name
        self.depends_on: List[str] = list(depends_on or [])
        self.ops: List[CommOp] = []
        self.completed = False

    def _add(self, kind: CommOpType, tensor: torch.Tensor, **kwargs) -> "CommPhase":
        self.ops.append(CommOp(kind, tensor, kwargs))
        return self

    def allreduce(self, tensor, **kw): return self._add(CommOpType.ALLREDUCE, tensor, **kw)
    def allgather(self, tensor, **kw): return self._add(CommOpType.ALLGATHER, tensor, **kw)
    def reduce_scatter(self, tensor, **kw): return self._add(CommOpType.REDUCE_SCATTER, tensor, **kw)
    def send(self, tensor, dst: int, **kw): return self._add(CommOpType.SEND, tensor, dst=dst, **kw)
    def recv(self, tensor, src: int, **kw): return self._add(CommOpType.RECV, tensor, src=src, **kw)
    def all_to_all(self, tensor, **kw): return self._add(CommOpType.ALL_TO_ALL, tensor, **kw)


class CommScheduler:
    def __init__(self, num_sms: int = 32):
        self.num_sms = num_sms
        self.phases: Dict[str, CommPhase] = {}
        self._order: List[str] = []
        self._compiled = False

    def phase(self, name: str, depends_on: Optional[List[str]] = None) -> CommPhase:
        if name in self.phases:
            raise ValueError(f"phase {name!r} already exists")
        p = CommPhase(name, depends_on)
        self.phases[name] = p
        self._compiled = False
        return p

    def compile(self) -> "CommScheduler":
        order: List[str] = []
        state: Dict[str, int] = {}

        def visit(name: str, trail: List[str]) -> None:
            if name not in self.phases:
                raise ValueError(f"phase {trail[-1] if trail else '?'!r} depends on unknown phase {name!r}")
            s = state.get(name, 0)
            if s == 2:
                return
            if s == 1:
                raise ValueError("cyclic dependency between communication phases: " + " -> ".join(trail + [name]))
            state[name] = 1
            for dep in self.phases[name].depends_on:
                visit(dep, trail + [name])
            state[name] = 2
            order.append(name)

        for name in self.phases:
            visit(name, [])
        self._order = order
        self._compiled = True
        return self

    def execute(self, async_mode: bool = False) -> None:
        if not self._compiled:
            self.compile()
        for name in self._order:
            ph = self.phases[name]
            for dep in ph.depends_on:
                self._wait_phase(self.phases[dep])
            for op in ph.ops:
                self._issue(op, async_mode)
            if not async_mode:
                self._wait_phase(ph)

    def _issue(self, op: CommOp, async_mode: bool) -> None:
        kw = dict(op.kwargs)
        t = op.op_type
        if t == CommOpType.ALLREDUCE:
            r = patterns.allreduce(op.tensor, async_op=async_mode, **kw)
        elif t == CommOpType.ALLGATHER:
            r = patterns.allgather(op.tensor, async_op=async_mode, **kw)
        elif t == CommOpType.REDUCE_SCATTER:
            r = patterns.reduce_scatter(op.tensor, async_op=async_mode, **kw)
        elif t == CommOpType.SEND:
            r = patterns.send(op.tensor, async_op=async_mode, **kw)
        elif t == CommOpType.RECV:
            r = patterns.recv(op.tensor, async_op=async_mode, **kw)
        elif t == CommOpType.ALL_TO_ALL:
            r = patterns.all_to_all(op.tensor, async_op=async_mode, **kw)
        else:
            raise ValueError(f"unsupported op {t}")
        if async_mode and hasattr(r, "wait"):
            op.handle = r
        else:
            op.result = r

    def _wait_phase(self, ph: CommPhase) -> None:
        for op in ph.ops:
            if op.handle is not None:
                op.result = op.handle.wait()
                op.handle = None
        ph.completed = True

    def wait_all(self) -> None:
        for ph in self.phases.values():
            self._wait_phase(ph)

    def reset(self) -> None:
        self.phases.clear()
        self._order = []
        self._compiled = False

    def get_schedule_info(self) -> Dict[str, Any]:
        return {
            "num_sms": self.num_sms,
            "num_phases": len(self.phases),
            "order": list(self._order),
            "phases": {n: {"depends_on": p.depends_on, "ops": [o.op_type.value for o in p.ops]}
                       for n, p in self.phases.items()},
        }
