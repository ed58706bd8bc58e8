"""Execution contexts: ``Context`` for ad-hoc compute + all-reduce, ``PersistentContext`` for a module.

API of the reference's maco/core/context.py:31-243. The reference's ``PersistentContext`` only
validates the SM split and calls the module; here it also records which tensors were registered
and exposes the validated role split that a persistent launch uses.
"""
from __future__ import annotations

from typing import Any, Callable, List, Optional

import torch
import torch.distributed as dist

from .sm_manager import SMConfig, SMManager
from .tensor_registry import TensorRegistry


class _AsyncResult:
    def __init__(self, tensor: torch.Tensor, handle):
        self.tensor, self.handle = tensor, handle

    def wait(self) -> torch.Tensor:
        if self.handle is not None:
            self.handle.wait()
            self.handle = None
        return self.tensor

    def is_completed(self) -> bool:
        return self.handle is None or self.handle.is_completed()


class Context:
    def __init__(self, world_size: int = 1, compute_sms: Optional[int] = None, comm_sms: Optional[int] = None,
                 overlap: bool = True):
        self.world_size = world_size
        self.compute_sms = compute_sms
        self.comm_sms = comm_sms
        self.overlap = overlap
        self._pending: List[_AsyncResult] = []

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self._flush()
        return False

    def compute(self, fn: Callable, *args, **kwargs) -> Any:
        return fn(*args, **kwargs)

    def allreduce(self, tensor: torch.Tensor, op: str = "sum", async_op: Optional[bool] = None):
        from ..comm import patterns
        async_op = self.overlap if async_op is None else async_op
        if self.world_size <= 1 or not (dist.is_available() and dist.is_initialized()):
            return tensor
        if async_op:
            h = patterns.allreduce(tensor, op=op, async_op=True)
            res = _AsyncResult(tensor, h)
            self._pending.append(res)
            return res
        return patterns.allreduce(tensor, op=op)

    def _flush(self) -> None:
        for r in self._pending:
            r.wait()
        self._pending.clear()


class PersistentContext:
    def __init__(self, model=None, sm_config: Optional[SMConfig] = None):
        self.model = model
        self.sm_manager = SMManager(sm_config) if sm_config is not None or torch.cuda.is_available() else None
        self.registry = TensorRegistry()
        self.worker_config: Optional[dict] = None
        self._active = False

    def __enter__(self):
        self._compile()
        self._active = True
        return self

    def __exit__(self, exc_type, exc, tb):
        self._cleanup()
        return False

    def _compile(self) -> None:
        if self.sm_manager is not None:
            self.worker_config = self.sm_manager.get_worker_config()

    def _cleanup(self) -> None:
        self._active = False

    def forward(self, *args, **kwargs):
        if self.model is None:
            raise RuntimeError("PersistentContext has no model")
        return self.model(*args, **kwargs)

    __call__ = forward

    def register_tensor(self, tensor: torch.Tensor, name: str, is_weight: bool = False):
        return self.registry.register(tensor, name, is_weight=is_weight, is_input=not is_weight)

    def register_output(self, shape, name: str, dtype: torch.dtype = torch.float32, device=None):
        return self.registry.register_output(shape, name, dtype=dtype, device=device)
