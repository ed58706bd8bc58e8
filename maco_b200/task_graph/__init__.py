"""Task graph front end, schedule and runtimes (reference: maco/task_graph/__init__.py)."""
from .exceptions import (
    AlreadyCompiledError,
    CompilationError,
    CUDANotAvailableError,
    CyclicDependencyError,
    DeviceError,
    DimensionError,
    DTypeMismatchError,
    MacoTimeoutError,
    NotCompiledError,
    NullInputError,
    PeerLostError,
    RuntimeError,
    ShapeMismatchError,
    TaskGraphError,
    ValidationError,
)
from .graph import TaskGraph
from .nodes import OverlapGroup, TaskNode, TaskType
from .overlap_scheduler import OverlapMode, OverlapPlan, OverlapRuntime, OverlapScheduler
from .runtime import MacoRuntime, PersistentRuntime, ReferenceRuntime, StreamRuntime
from .schedule import TaskSchedule
from .validation import (
    infer_device,
    infer_dtype,
    validate_dtype_match,
    validate_linear_shapes,
    validate_matmul_shapes,
    validate_same_device,
    validate_tensor,
)

__all__ = [
    "TaskGraph", "TaskNode", "TaskType", "OverlapGroup", "TaskSchedule",
    "TaskGraphError", "ValidationError", "NullInputError", "DeviceError", "ShapeMismatchError", "DimensionError",
    "DTypeMismatchError", "CompilationError", "CyclicDependencyError", "NotCompiledError", "AlreadyCompiledError",
    "RuntimeError", "CUDANotAvailableError", "MacoTimeoutError", "PeerLostError",
    "validate_tensor", "validate_linear_shapes", "validate_matmul_shapes", "validate_dtype_match",
    "validate_same_device", "infer_device", "infer_dtype",
    "StreamRuntime", "MacoRuntime", "PersistentRuntime", "ReferenceRuntime",
    "OverlapScheduler", "OverlapPlan", "OverlapMode", "OverlapRuntime",
]
