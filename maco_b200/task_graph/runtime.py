"""Executors of a compiled TaskGraph.

* ``ReferenceRuntime`` - plain PyTorch ops on any device plus torch.distributed (gloo on CPU):
  the numerical oracle and the CPU path.
* ``StreamRuntime`` - one launch of this package's own CUDA kernels per node; overlap groups put
  their communication on the comm stream behind per-wave events. This is the shape of the
  reference's live runtime (maco/task_graph/runtime.py:160-234), with the kernels replaced and
  the overlap metadata honoured.
* ``PersistentRuntime`` - lowers the graph to tile-granular tasks and runs them in ONE launch of
  the persistent task kernel (scheduler CTA + worker CTAs). This is what the reference's
  ``MacoRuntime`` (runtime.py:21-144) was meant to be and never was: it is never instantiated
  there, passes one input and one dependency per task, and re-uploads every task with three host
  syncs. Here the task table is built once at compile() and uploaded in one copy.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .exceptions import MacoTimeoutError
from .nodes import TaskNode, TaskType
from .schedule import TaskSchedule


def _world() -> int:
    from ..comm.process_group import get_world_size
    return get_world_size()


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-rotation rotary embedding on [tokens, heads, head_dim] in fp32."""
    d = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d], xf[..., d:]
    c, s = cos.float().unsqueeze(1), sin.float().unsqueeze(1)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def rmsnorm_reference(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class _RuntimeBase:
    def __init__(self, device: torch.device, graph=None):
        self.device = torch.device(device)
        self.graph = graph

    # ---- communication nodes (shared) ----------------------------------------------------
    def _execute_allreduce(self, node: TaskNode) -> None:
        if _world() == 1:
            return
        from ..comm import patterns
        patterns.allreduce(node.outputs[0], op=node.attrs.get("op", "sum"))

    def _execute_allgather(self, node: TaskNode) -> None:
        src, out = node.inputs[0], node.outputs[0]
        if _world() == 1:
            out.copy_(src)
            return
        dist.all_gather_into_tensor(out, src.contiguous())

    def _execute_reduce_scatter(self, node: TaskNode) -> None:
        src, out = node.inputs[0], node.outputs[0]
        if _world() == 1:
            out.copy_(src)
            return
        from ..comm import patterns
        out.copy_(patterns.reduce_scatter(src, op=node.attrs.get("op", "sum")))

    def _execute_broadcast(self, node: TaskNode) -> None:
        if _world() > 1:
            dist.broadcast(node.outputs[0], src=node.attrs.get("src", 0))

    def _execute_all_to_all(self, node: TaskNode) -> None:
        src, out = node.inputs[0], node.outputs[0]
        if _world() == 1:
            out.copy_(src)
            return
        from ..comm import patterns
        sd, gd = node.attrs.get("scatter_dim", 0), node.attrs.get("gather_dim", 0)
        if sd == gd == 0:
            patterns.all_to_all_single(out, src)
        elif src.dim() == 4:
            out.copy_(patterns.all_to_all_4D(src, sd, gd))
        else:
            out.copy_(patterns.all_to_all(src, sd, gd))

    def _execute_custom(self, node: TaskNode) -> None:
        result = node.custom_fn(*node.inputs)
        if result is not None and node.outputs:
            if isinstance(result, (tuple, list)):
                for o, r in zip(node.outputs, result):
                    if r is not o:
                        o.copy_(r)
            elif result is not node.outputs[0]:
                node.outputs[0].copy_(result)

    def _execute_comm(self, node: TaskNode) -> bool:
        t = node.task_type
        if t == TaskType.ALLREDUCE:
            self._execute_allreduce(node)
        elif t == TaskType.ALLGATHER:
            self._execute_allgather(node)
        elif t == TaskType.REDUCE_SCATTER:
            self._execute_reduce_scatter(node)
        elif t == TaskType.BROADCAST:
            self._execute_broadcast(node)
        elif t == TaskType.ALL_TO_ALL:
            self._execute_all_to_all(node)
        elif t in (TaskType.CUSTOM_COMM, TaskType.CUSTOM_COMPUTE):
            self._execute_custom(node)
        elif t in (TaskType.NOP, TaskType.PEER_BARRIER):
            pass
        else:
            return False
        return True


class ReferenceRuntime(_RuntimeBase):
    """Plain PyTorch execution in schedule order."""

    def execute(self, schedule: TaskSchedule, stream=None) -> None:
        for wave in schedule.waves:
            for node in wave:
                self._execute_task(node)

    def _execute_task(self, node: TaskNode) -> None:
        if self._execute_comm(node):
            return
        t, ins, out = node.task_type, node.inputs, node.outputs[0]
        if out.numel() == 0:
            return
        if t == TaskType.LINEAR:
            x, w = ins[0], ins[1]
            b = ins[2] if node.attrs.get("has_bias") else None
            y = torch.nn.functional.linear(x, w, b)
            act = node.attrs.get("activation")
            if act == "gelu":
                y = torch.nn.functional.gelu(y, approximate="tanh")
            elif act == "silu":
                y = torch.nn.functional.silu(y)
            elif act == "swiglu":
                n = y.shape[-1]
                yv = y.reshape(*y.shape[:-1], n // 256, 2, 128)
                y = (torch.nn.functional.silu(yv[..., 0, :].float()) * yv[..., 1, :].float()).to(y.dtype)
                y = y.reshape(*out.shape)
            out.copy_(y)
        elif t == TaskType.MATMUL:
            torch.mm(ins[0], ins[1], out=out)
        elif t == TaskType.GELU:
            out.copy_(torch.nn.functional.gelu(ins[0].float(), approximate="tanh").to(out.dtype))
        elif t == TaskType.SILU:
            out.copy_(torch.nn.functional.silu(ins[0].float()).to(out.dtype))
        elif t == TaskType.SOFTMAX:
            out.copy_(torch.softmax(ins[0].float(), dim=-1).to(out.dtype))
        elif t == TaskType.SCALE:
            out.copy_((ins[0].float() * node.attrs["factor"]).to(out.dtype))
        elif t == TaskType.ADD:
            out.copy_((ins[0].float() + ins[1].float()).to(out.dtype))
        elif t == TaskType.SILU_GATE:
            out.copy_((torch.nn.functional.silu(ins[0].float()) * ins[1].float()).to(out.dtype))
        elif t == TaskType.RMSNORM:
            out.copy_(rmsnorm_reference(ins[0], ins[1], node.attrs["eps"]))
        elif t == TaskType.LAYERNORM:
            out.copy_(torch.nn.functional.layer_norm(ins[0].float(), (ins[0].shape[-1],), ins[1].float(),
                                                     ins[2].float(), node.attrs["eps"]).to(out.dtype))
        elif t == TaskType.ROPE:
            out.copy_(rope_reference(ins[0], ins[1], ins[2]))
        else:
            raise NotImplementedError(f"ReferenceRuntime has no implementation for {t.name}")


class StreamRuntime(_RuntimeBase):
    """One kernel launch per node with this package's CUDA operators."""

    def __init__(self, device, graph=None):
        super().__init__(device, graph)
        from ..sync.stream_manager import StreamManager
        self._sm = StreamManager(self.device) if self.device.type == "cuda" else None

    def execute(self, schedule: TaskSchedule, stream=None) -> None:
        if stream is not None and isinstance(stream, torch.cuda.Stream):
            with torch.cuda.stream(stream):
                self._run(schedule)
        else:
            self._run(schedule)

    def _run(self, schedule: TaskSchedule) -> None:
        main = torch.cuda.current_stream(self.device)
        comm_stream = self._sm.comm_stream
        done: Dict[int, torch.cuda.Event] = {}      # node id -> completion event of an off-stream node
        forked = False
        from ..config import config
        overlap_on = str(config.overlap_strategy).lower() != "none"      # "none": everything on the main stream
        for wave in schedule.waves:
            for node in wave:
                off = overlap_on and node.is_comm and node._overlap_role == "comm" and _world() > 1
                target = comm_stream if off else main
                for dep in node.depends_on:
                    ev = done.get(dep._node_id)
                    if ev is not None:
                        target.wait_event(ev)
                if off:
                    # wait for everything issued so far on the main stream that this node depends on
                    ev = torch.cuda.Event()
                    ev.record(main)
                    comm_stream.wait_event(ev)
                    with torch.cuda.stream(comm_stream):
                        self._execute_task(node)
                        fin = torch.cuda.Event()
                        fin.record(comm_stream)
                    done[node._node_id] = fin
                    forked = True
                else:
                    self._execute_task(node)
        if forked:
            for ev in done.values():
                main.wait_event(ev)

    def _execute_task(self, node: TaskNode) -> None:
        if self._execute_comm(node):
            return
        from .. import ops
        t, ins, out = node.task_type, node.inputs, node.outputs[0]
        if out.numel() == 0:
            return
        if t == TaskType.LINEAR:
            b = ins[2] if node.attrs.get("has_bias") else None
            ops.linear(ins[0], ins[1], b, out=out, epilogue=node.attrs.get("activation"))
        elif t == TaskType.MATMUL:
            ops.matmul(ins[0], ins[1], out=out)
        elif t == TaskType.GELU:
            ops.gelu(ins[0], out=out)
        elif t == TaskType.SILU:
            ops.silu(ins[0], out=out)
        elif t == TaskType.SOFTMAX:
            ops.softmax(ins[0], out=out)
        elif t == TaskType.SCALE:
            ops.scale(ins[0], node.attrs["factor"], out=out)
        elif t == TaskType.ADD:
            ops.add(ins[0], ins[1], out=out)
        elif t == TaskType.SILU_GATE:
            ops.silu_gate(ins[0], ins[1], out=out)
        elif t == TaskType.RMSNORM:
            ops.rmsnorm(ins[0], ins[1], node.attrs["eps"], out=out)
        elif t == TaskType.LAYERNORM:
            ops.layernorm(ins[0], ins[1], ins[2], node.attrs["eps"], out=out)
        elif t == TaskType.ROPE:
            ops.rope(ins[0], ins[1], ins[2], out=out)
        else:
            raise NotImplementedError(f"StreamRuntime has no implementation for {t.name}")


def _schedule_key(graph) -> tuple:
    """Identity of a compiled schedule: node types and attributes, the address / shape / strides / dtype of every
    tensor (task descriptors carry absolute addresses), the dependency structure, and everything else the lowering
    reads (world, rank, device architecture, worker count, scheduling mode, debug / trace switches)."""
    import os
    from ..comm.process_group import get_rank, get_world_size
    from ..config import config

    def tkey(t):
        return (t.data_ptr(), tuple(t.shape), tuple(t.stride()), str(t.dtype))

    nodes = []
    for n in graph._nodes:
        attrs = tuple(sorted((k, v if isinstance(v, (int, float, str, bool, type(None))) else repr(v)) for k, v in n.attrs.items()))
        nodes.append((int(n.task_type), attrs, tuple(tkey(t) for t in n.inputs), tuple(tkey(t) for t in n.outputs),
                      tuple(d._node_id for d in n.depends_on), n._wave_id, n._overlap_role))
    cap = torch.cuda.get_device_capability(graph.device)
    smc = getattr(graph, "sm_config", None)
    return (tuple(nodes), get_world_size(), get_rank(), str(graph.device), cap, graph.num_workers,
            os.environ.get("MACO_PERSISTENT_MODE", "static"), bool(config.debug), bool(config.profile), str(config.sm_policy),
            repr(smc.to_dict()) if smc is not None else None)


class PersistentRuntime(_RuntimeBase):
    """Runs the graph as tile tasks inside one launch of the persistent task kernel.

    Compiled programs are cached per process (least recently used first out, ``SCHEDULE_CACHE_SIZE`` entries) under
    ``_schedule_key``: code that rebuilds the same graph over the same tensors every step (the reference's examples
    do) pays the lowering, thousands of descriptors for a large layer, once. A cached program keeps its tensors
    alive, so the addresses in its descriptors stay valid. Programs over the symmetric heap are not cached: their
    stand-in buffers and event tables come from a collective allocation sequence."""

    SCHEDULE_CACHE_SIZE = 32
    _cache: "OrderedDict[tuple, object]" = None
    cache_hits = 0

    def __init__(self, graph):
        super().__init__(graph.device, graph)
        from collections import OrderedDict
        from ..ops import megakernel
        cls = PersistentRuntime
        if cls._cache is None:
            cls._cache = OrderedDict()
        key = _schedule_key(graph)
        prog = cls._cache.get(key)
        if prog is not None:
            cls._cache.move_to_end(key)
            cls.cache_hits += 1
        else:
            prog = megakernel.lower_graph(graph)
            if prog.heap is None:
                cls._cache[key] = prog
                while len(cls._cache) > cls.SCHEDULE_CACHE_SIZE:
                    cls._cache.popitem(last=False)
        self._program = prog

    @classmethod
    def clear_schedule_cache(cls) -> None:
        if cls._cache is not None:
            cls._cache.clear()

    @staticmethod
    def can_run(graph) -> bool:
        if graph.device.type != "cuda" or not torch.cuda.is_available():
            return False
        try:
            from ..ops import megakernel
        except Exception:
            return False
        return megakernel.can_lower(graph)

    def execute(self, schedule: TaskSchedule, stream=None) -> None:
        self._program.run(stream=stream)

    def describe(self) -> str:
        return self._program.describe()

    def stats(self) -> dict:
        return self._program.stats()


# Name kept for code written against the reference, where MacoRuntime is the persistent-kernel runtime.
MacoRuntime = PersistentRuntime
