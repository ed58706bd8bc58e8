"""Communication layer: process groups, library collectives (NCCL / gloo), patterns, phase
scheduler, and the peer-memory backend (the NVSHMEM-style symmetric heap of this package).

Re-exports what the reference's maco/comm/__init__.py:8-45 exports.
"""
from . import patterns
from .nccl_backend import CommHandle, NCCLBackend, OverlapMode, get_backend, init_backend
from .nccl_ops import (
    AsyncHandle,
    async_all_gather,
    async_all_reduce,
    async_all_to_all,
    async_all_to_all_4d,
    async_broadcast,
    sync_stream,
    wait_comm_stream,
)
from .peer_backend import (
    finalize_nvshmem,
    init_nvshmem,
    is_nvshmem_available,
    nvshmem_all_to_all_4D,
    nvshmem_allreduce,
    nvshmem_barrier,
    nvshmem_my_pe,
    nvshmem_n_pes,
)
from .process_group import (
    ProcessGroupManager,
    barrier,
    get_local_rank,
    get_rank,
    get_world_size,
    is_initialized,
)
from .scheduler import CommOp, CommOpType, CommPhase, CommScheduler

__all__ = [
    "ProcessGroupManager", "get_world_size", "get_rank", "get_local_rank", "is_initialized", "barrier",
    "AsyncHandle", "async_all_reduce", "async_all_gather", "async_all_to_all", "async_all_to_all_4d",
    "async_broadcast", "sync_stream", "wait_comm_stream", "patterns", "NCCLBackend", "OverlapMode", "CommHandle",
    "get_backend", "init_backend", "CommScheduler", "CommPhase", "CommOp", "CommOpType",
    "is_nvshmem_available", "init_nvshmem", "finalize_nvshmem", "nvshmem_my_pe", "nvshmem_n_pes",
    "nvshmem_barrier", "nvshmem_allreduce", "nvshmem_all_to_all_4D",
]
