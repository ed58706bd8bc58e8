"""Exception hierarchy of the task graph.

Same class names, attributes and inheritance as the reference's
maco/task_graph/exceptions.py:8-137, so ``except`` clauses written against it keep working.
Every message names the offending parameter / method and ends with a ``Hint:`` line.
"""
from __future__ import annotations

from typing import Optional, Sequence


class TaskGraphError(Exception):
    """Root of every error the task graph raises."""


class ValidationError(TaskGraphError):
    """An argument of a graph-building call is unusable."""


class NullInputError(ValidationError):
    def __init__(self, param_name: str, method_name: str):
        self.param_name = param_name
        self.method_name = method_name
        super().__init__(
            f"'{param_name}' cannot be None in {method_name}()\n"
            f"Hint: pass an initialised tensor as '{param_name}' to graph.{method_name}()"
        )


class DeviceError(ValidationError):
    def __init__(self, param_name: str, actual_device: str, expected_device: str = "cuda"):
        self.param_name = param_name
        self.actual_device = actual_device
        self.expected_device = expected_device
        super().__init__(
            f"'{param_name}' is on {actual_device}, expected {expected_device}\n"
            f"Hint: move it with tensor.to('{expected_device}') or build the graph for that device"
        )


class ShapeMismatchError(ValidationError):
    def __init__(self, op: str, details: str, hint: Optional[str] = None):
        self.op = op
        self.details = details
        msg = f"Shape mismatch in '{op}': {details}"
        if hint:
            msg += f"\nHint: {hint}"
        super().__init__(msg)


class DimensionError(ValidationError):
    def __init__(self, param_name: str, expected_ndim, actual_ndim: int):
        self.param_name = param_name
        self.expected_ndim = expected_ndim
        self.actual_ndim = actual_ndim
        super().__init__(
            f"'{param_name}' has {actual_ndim} dimensions, expected {expected_ndim}\n"
            f"Hint: reshape '{param_name}' so that it has {expected_ndim} dimensions"
        )


class DTypeMismatchError(ValidationError):
    def __init__(self, param1: str, dtype1, param2: str, dtype2):
        self.param1, self.dtype1, self.param2, self.dtype2 = param1, dtype1, param2, dtype2
        super().__init__(
            f"dtype mismatch: '{param1}' is {dtype1}, '{param2}' is {dtype2}\n"
            f"Hint: convert one of them with tensor.to(dtype) so both agree"
        )


class CompilationError(TaskGraphError):
    """compile() could not produce a schedule."""


class CyclicDependencyError(CompilationError):
    def __init__(self, cycle_nodes: Optional[Sequence] = None):
        self.cycle_nodes = list(cycle_nodes) if cycle_nodes else None
        msg = "Cyclic dependency detected in task graph"
        if self.cycle_nodes:
            msg += ": " + " -> ".join(str(n) for n in self.cycle_nodes)
        msg += "\nHint: look at the add_dependency() / depends_on edges and drop the one that closes the loop"
        super().__init__(msg)


class NotCompiledError(TaskGraphError):
    def __init__(self):
        super().__init__("TaskGraph has not been compiled\nHint: call graph.compile() before graph.execute()")


class AlreadyCompiledError(TaskGraphError):
    def __init__(self):
        super().__init__(
            "Cannot modify TaskGraph after compilation\n"
            "Hint: build a new TaskGraph for a different set of operations"
        )


class RuntimeError(TaskGraphError):  # noqa: A001 - the reference exports this name from the package
    """Failure while a compiled graph executes."""


class CUDANotAvailableError(RuntimeError):
    def __init__(self):
        super().__init__("CUDA is not available\nHint: a CUDA build of PyTorch and a visible GPU are required")


class MacoTimeoutError(RuntimeError):
    """A bounded device-side wait ran out (a producer never signalled)."""

    def __init__(self, detail: str = ""):
        self.detail = detail
        super().__init__(
            "A device-side wait exceeded its time budget" + (f": {detail}" if detail else "") +
            "\nHint: a producer task or a peer rank never signalled; the kernel returned and the context is usable"
        )


class PeerLostError(RuntimeError):
    """A peer rank stopped answering (heartbeat or collective timeout)."""

    def __init__(self, rank: int = -1, detail: str = ""):
        self.rank = rank
        super().__init__(
            f"Peer rank {rank} is not responding" + (f": {detail}" if detail else "") +
            "\nHint: re-rendezvous with the surviving ranks and recompile the graph for the new world size"
        )
