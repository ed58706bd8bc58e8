"""maco_b200: SM-level task scheduling and compute/communication overlap for B200 (sm_100a).

Top-level API of the reference package (maco/__init__.py:70-415): ``init`` / ``cleanup``, rank and
world-size getters, the stream-overlap convenience calls, and re-exports of the task graph, comm,
sync, overlap and core layers. ``import maco_b200 as maco`` is the intended drop-in spelling.
"""
from __future__ import annotations

import logging
import os
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist

from . import comm, core, overlap, sync, task_graph
from .comm import (
    AsyncHandle,
    CommScheduler,
    NCCLBackend,
    ProcessGroupManager,
    async_all_gather,
    async_all_reduce,
    async_all_to_all,
    async_all_to_all_4d,
    async_broadcast,
    finalize_nvshmem,
    init_nvshmem,
    is_nvshmem_available,
    nvshmem_all_to_all_4D,
    nvshmem_allreduce,
    nvshmem_barrier,
    nvshmem_my_pe,
    nvshmem_n_pes,
    patterns,
    sync_stream,
    wait_comm_stream,
)
from .comm.nccl_backend import OverlapMode as BackendOverlapMode
from .comm.nccl_backend import get_backend, init_backend
from .config import MacoConfig, config
from .core import Context, PersistentContext, Role, SMConfig, SMManager, TensorRegistry, auto_config
from .overlap import OverlapManager, OverlapRegion
from .sync import (
    DeviceSignal,
    OverlapContext,
    Signal,
    SignalWait,
    StreamManager,
    create_signal,
)
from .task_graph import (
    AlreadyCompiledError,
    CyclicDependencyError,
    DeviceError,
    DimensionError,
    DTypeMismatchError,
    MacoTimeoutError,
    NotCompiledError,
    NullInputError,
    OverlapGroup,
    OverlapMode,
    OverlapPlan,
    OverlapRuntime,
    OverlapScheduler,
    PeerLostError,
    ShapeMismatchError,
    TaskGraph,
    TaskGraphError,
    TaskNode,
    TaskSchedule,
    TaskType,
    ValidationError,
)

__version__ = "0.1.0"

log = logging.getLogger("maco_b200")

_initialized = False
_overlap_manager: Optional[OverlapManager] = None
_rank = 0
_world_size = 1


def init(backend: str = "nccl", rank: Optional[int] = None, world_size: Optional[int] = None,
         init_method: Optional[str] = None, overlap_mode: str = "stream", peer_heap: Optional[bool] = None,
         timeout_s: Optional[float] = None) -> None:
    """Initialises the process group (from RANK / LOCAL_RANK / WORLD_SIZE when not given), picks the
    device, builds the global overlap manager and library backend, and - on CUDA with more than
    one rank and ``config.backend == "peer"`` - the symmetric heap for in-kernel collectives."""
    global _initialized, _overlap_manager, _rank, _world_size
    if _initialized:
        return
    pgm = ProcessGroupManager()
    pgm.init_process_group(backend=backend, init_method=init_method, world_size=world_size, rank=rank,
                           timeout_s=timeout_s)
    _rank, _world_size = pgm.rank, pgm.world_size
    _overlap_manager = OverlapManager(pgm.device if pgm.device.type == "cuda" else None)
    mode = {"none": BackendOverlapMode.NONE, "stream": BackendOverlapMode.STREAM,
            "persistent": BackendOverlapMode.PERSISTENT}.get(str(overlap_mode).lower(), BackendOverlapMode.STREAM)
    init_backend(rank=_rank, world_size=_world_size, overlap_mode=mode)
    want_heap = peer_heap if peer_heap is not None else (config.backend == "peer")
    if want_heap and _world_size > 1 and pgm.device.type == "cuda":
        init_nvshmem()
    _initialized = True
    if config.verbose and _rank == 0:
        log.info("initialised: world=%d backend=%s device=%s", _world_size, pgm.backend, pgm.device)


def cleanup(abort: bool = False) -> None:
    """Tears down the heap, the overlap manager and the process group. ``abort=True`` is the path after
    a peer was lost: nothing collective is attempted (no barrier, no graceful group shutdown)."""
    global _initialized, _overlap_manager
    if _overlap_manager is not None:
        _overlap_manager.sync_streams()
    try:
        finalize_nvshmem(collective=not abort)
    except Exception:
        pass
    m = ProcessGroupManager._instance
    if m is not None:
        if abort:
            ProcessGroupManager._instance = None
        else:
            m.destroy()
    _overlap_manager = None
    _initialized = False


def recover(lost_ranks, port: Optional[int] = None, backend: Optional[str] = None,
            timeout_s: Optional[float] = None):
    """Elastic recovery after ``PeerLostError``: tears this rank's state down without any collective (heap, cached
    programs, process group), then rendezvouses again with the SURVIVORS only. Ranks are renumbered in their old
    order (the lowest surviving rank becomes rank 0 and hosts the new rendezvous store, on ``port`` or the old
    master port + 1 + number of recoveries so far). Graphs and programs must be rebuilt afterwards: their task
    tables name the old world. Returns (new_rank, new_world_size).

    Every survivor calls it with the same ``lost_ranks`` (they learn them from the same heartbeats). The reference
    has no failure path at all (maco/__init__.py:262-273 only destroys the group)."""
    global _recoveries
    import os
    pgm = ProcessGroupManager._instance
    old_rank, old_world = (pgm.rank, pgm.world_size) if pgm is not None else (_rank, _world_size)
    be = backend or (pgm.backend if pgm is not None else None) or "gloo"
    lost = sorted(set(int(r) for r in lost_ranks))
    if old_rank in lost:
        raise ValueError("a rank that is counted as lost cannot take part in the recovery")
    survivors = [r for r in range(old_world) if r not in lost]
    cleanup(abort=True)
    try:
        import torch.distributed as _dist
        if _dist.is_initialized():
            _dist.destroy_process_group()
    except Exception:
        pass
    _recoveries += 1
    new_rank, new_world = survivors.index(old_rank), len(survivors)
    new_port = int(port) if port is not None else int(os.environ.get("MASTER_PORT", "29500")) + _recoveries
    os.environ.update({"RANK": str(new_rank), "WORLD_SIZE": str(new_world), "MASTER_PORT": str(new_port)})
    init(backend=be, rank=new_rank, world_size=new_world, timeout_s=timeout_s)
    return new_rank, new_world


_recoveries = 0


def get_rank() -> int:
    return comm.get_rank()


def get_world_size() -> int:
    return comm.get_world_size()


def is_initialized() -> bool:
    return _initialized


def get_overlap_manager() -> OverlapManager:
    global _overlap_manager
    if _overlap_manager is None:
        _overlap_manager = OverlapManager()
    return _overlap_manager


def overlap_compute_and_comm(compute_fn: Callable[[], Any], comm_tensor: torch.Tensor, comm_op: str = "allreduce", **kw):
    """Runs ``compute_fn`` while ``comm_tensor`` goes through ``comm_op``; returns (compute_result, comm_result)."""
    return get_overlap_manager().overlap_compute_and_comm(compute_fn, comm_tensor, comm_op, **kw)


def overlap_all_to_all_with_compute(all_to_all_fn: Callable[[], Any], compute_fn: Callable[[], Any]):
    return get_overlap_manager().overlap_all_to_all_with_compute(all_to_all_fn, compute_fn)


def overlap_region():
    return get_overlap_manager().overlap_region()


def get_comm_stream():
    return get_overlap_manager().get_comm_stream()


def get_compute_stream():
    return get_overlap_manager().get_compute_stream()


def sync_streams() -> None:
    get_overlap_manager().sync_streams()


__all__ = [
    "init", "cleanup", "recover", "get_rank", "get_world_size", "is_initialized", "config", "MacoConfig",
    "get_overlap_manager", "overlap_compute_and_comm", "overlap_all_to_all_with_compute", "overlap_region",
    "get_comm_stream", "get_compute_stream", "sync_streams",
    "TaskGraph", "TaskNode", "TaskType", "OverlapGroup", "TaskSchedule", "OverlapScheduler", "OverlapPlan",
    "OverlapMode", "OverlapRuntime",
    "TaskGraphError", "ValidationError", "NullInputError", "DeviceError", "ShapeMismatchError", "DimensionError",
    "DTypeMismatchError", "CyclicDependencyError", "NotCompiledError", "AlreadyCompiledError", "MacoTimeoutError",
    "PeerLostError",
    "ProcessGroupManager", "AsyncHandle", "async_all_reduce", "async_all_gather", "async_all_to_all",
    "async_all_to_all_4d", "async_broadcast", "sync_stream", "wait_comm_stream", "patterns", "NCCLBackend",
    "CommScheduler", "get_backend", "init_backend",
    "is_nvshmem_available", "init_nvshmem", "finalize_nvshmem", "nvshmem_my_pe", "nvshmem_n_pes", "nvshmem_barrier",
    "nvshmem_allreduce", "nvshmem_all_to_all_4D",
    "StreamManager", "Signal", "SignalWait", "create_signal", "OverlapContext", "DeviceSignal",
    "OverlapManager", "OverlapRegion",
    "SMConfig", "SMManager", "Role", "auto_config", "Context", "PersistentContext", "TensorRegistry",
]
