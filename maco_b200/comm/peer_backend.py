"""Device-initiated communication backend: the role NVSHMEM plays in the reference.

The reference ships an optional NVSHMEM + MPI extension (maco/csrc/nvshmem_ops.cu, wrapped by
maco/comm/nvshmem_backend.py:28-249). Here the same entry points are served by this package's
own symmetric heap (peer-mapped device memory over NVLink, see ``maco_b200.parallel.symm_heap``)
and its in-kernel collectives; no NVSHMEM or MPI is needed. The function names are kept so code
written against the reference keeps importing.
"""
from __future__ import annotations

from typing import Optional

import torch

from .process_group import get_rank, get_world_size


def is_nvshmem_available() -> bool:
    """True when device-initiated peer communication can be used (CUDA + the native library)."""
    if not torch.cuda.is_available():
        return False
    from .. import _native
    return _native.available()


def init_nvshmem(heap_bytes: Optional[int] = None) -> bool:
    """Creates the symmetric heap over the current process group. Returns False when unavailable."""
    if not is_nvshmem_available():
        return False
    from ..parallel import symm_heap
    symm_heap.init_heap(heap_bytes)
    return True


def finalize_nvshmem(collective: bool = True) -> None:
    from ..parallel import symm_heap
    symm_heap.destroy_heap(collective=collective)


def nvshmem_my_pe() -> int:
    return get_rank()


def nvshmem_n_pes() -> int:
    return get_world_size()


def nvshmem_barrier() -> None:
    from ..parallel import collectives, symm_heap
    if symm_heap.current_heap() is not None and get_world_size() > 1:
        collectives.device_barrier()
    else:
        from .process_group import barrier
        barrier()


def nvshmem_allreduce(tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
    """All-reduce served by the in-kernel collective; copies through the heap if needed."""
    if op not in ("sum", "avg"):
        raise ValueError("the device-initiated all-reduce supports 'sum' and 'avg'")
    if get_world_size() == 1:
        return tensor
    from ..parallel import collectives
    return collectives.all_reduce_any(tensor, avg=(op == "avg"))


def nvshmem_all_to_all_4D(tensor: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1) -> torch.Tensor:
    if tensor.dim() != 4:
        raise ValueError("expected a 4-D tensor")
    if get_world_size() == 1:
        return tensor
    from ..parallel import collectives
    return collectives.all_to_all_4d_any(tensor, scatter_dim, gather_dim)


def nvshmem_allreduce_fallback(tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
    from . import patterns
    return patterns.allreduce(tensor, op=op)


def nvshmem_all_to_all_4D_fallback(tensor: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1) -> torch.Tensor:
    from . import patterns
    return patterns.all_to_all_4D(tensor, scatter_dim, gather_dim)
