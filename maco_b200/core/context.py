"""Execution contexts: ``Context`` for ad-hoc compute + all-reduce, ``PersistentContext`` for a module.

API of the reference's maco/core/context.py:31-243. The reference's ``PersistentContext`` only
validates the SM split and calls the module (``forward`` = ``model(*args)``, its ``register_*`` are TODOs). Here
``PersistentContext`` compiles the module into a ``TaskGraph`` when it is a chain of layers the kernel has tasks
for (``nn.Sequential`` / any module whose children run in order: Linear, GELU(tanh), SiLU, LayerNorm, RMSNorm,
Softmax, Identity, Dropout in eval mode): the forward pass of a given input shape is then ONE launch of the
persistent kernel with ``sm_config``'s compute SMs as workers, the weights are registered in the
``TensorRegistry``, and the graph is cached per input shape. Anything else falls back to calling the module.
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
        self._graphs: dict = {}                  # (shape, dtype, device) -> (graph, input buffer, output) or None
        self.last_runtime: Optional[str] = None  # "persistent" / "stream" / "reference" / "module" for the last forward

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

    # ------------------------------------------------------------------ module -> task graph
    def _layers(self):
        """The module's layers in execution order, or None when it is not a plain chain of supported layers."""
        import torch.nn as nn
        m = self.model
        if isinstance(m, nn.Sequential):
            mods = list(m)
        elif isinstance(m, (nn.Linear, nn.GELU, nn.SiLU, nn.LayerNorm, nn.Softmax)):
            mods = [m]
        else:
            return None
        ok = (nn.Linear, nn.GELU, nn.SiLU, nn.LayerNorm, nn.Softmax, nn.Identity, nn.Dropout)
        rms = getattr(nn, "RMSNorm", None)
        for x in mods:
            if not isinstance(x, ok) and not (rms is not None and isinstance(x, rms)):
                return None
            if isinstance(x, nn.GELU) and getattr(x, "approximate", "none") != "tanh":
                return None                      # the kernel's GELU is the tanh form
            if isinstance(x, nn.Dropout) and x.training and x.p > 0:
                return None
            if isinstance(x, nn.Softmax) and x.dim not in (-1, None):
                return None
        return mods

    def _graph_for(self, x: torch.Tensor):
        import torch.nn as nn
        from ..task_graph.graph import TaskGraph
        key = (tuple(x.shape), x.dtype, str(x.device))
        ent = self._graphs.get(key)
        if ent is not None:
            return ent
        mods = self._layers()
        if mods is None or not x.is_cuda:
            self._graphs[key] = None
            return None
        workers = self.worker_config["num_workers"] if self.worker_config else None
        g = TaskGraph(num_workers=workers, device=x.device)
        if self.sm_manager is not None:
            g.sm_config = self.sm_manager.config
        inp = torch.empty_like(x)
        cur = inp
        rms = getattr(nn, "RMSNorm", None)
        for i, m in enumerate(mods):
            if isinstance(m, nn.Linear):
                node = g.linear(cur, m.weight.detach(), m.bias.detach() if m.bias is not None else None, name=f"linear{i}")
                self.registry.register(m.weight.detach(), f"layer{i}.weight", is_weight=True)
            elif isinstance(m, nn.GELU):
                node = g.gelu(cur, name=f"gelu{i}")
            elif isinstance(m, nn.SiLU):
                node = g.silu(cur, name=f"silu{i}")
            elif isinstance(m, nn.LayerNorm):
                node = g.layernorm(cur, m.weight.detach(), m.bias.detach(), eps=m.eps, name=f"layernorm{i}")
            elif rms is not None and isinstance(m, rms):
                node = g.rmsnorm(cur, m.weight.detach(), eps=m.eps if m.eps is not None else torch.finfo(x.dtype).eps, name=f"rmsnorm{i}")
            elif isinstance(m, nn.Softmax):
                node = g.softmax(cur, name=f"softmax{i}")
            else:
                continue                         # Identity / inactive Dropout
            cur = node.output
        g.compile()
        ent = self._graphs[key] = (g, inp, cur)
        return ent

    def forward(self, *args, **kwargs):
        if self.model is None:
            raise RuntimeError("PersistentContext has no model")
        if len(args) == 1 and not kwargs and isinstance(args[0], torch.Tensor) and not torch.is_grad_enabled():
            ent = self._graph_for(args[0])
            if ent is not None:
                g, inp, out = ent
                inp.copy_(args[0])
                g.execute()
                self.last_runtime = g.runtime_kind
                return out
        self.last_runtime = "module"
        return self.model(*args, **kwargs)

    __call__ = forward

    def register_tensor(self, tensor: torch.Tensor, name: str, is_weight: bool = False):
        return self.registry.register(tensor, name, is_weight=is_weight, is_input=not is_weight)

    def register_output(self, shape, name: str, dtype: torch.dtype = torch.float32, device=None):
        return self.registry.register_output(shape, name, dtype=dtype, device=device)
