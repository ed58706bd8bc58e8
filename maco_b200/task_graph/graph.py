"""TaskGraph: build a DAG of tensor operations, compile it to a schedule, execute it.

Public surface of the reference's maco/task_graph/__init__.py:284-777 (``linear``, ``matmul``,
``custom``, ``allreduce``, ``all_to_all``, ``overlap``, ``compile``, ``execute``, ``summary``), plus the
built-in operators the persistent kernel runs natively (``rmsnorm``, ``layernorm``, ``gelu``, ``silu``,
``silu_gate``, ``softmax``, ``rope``, ``add``, ``scale``) and the collectives the reference's graph
lacks (``allgather``, ``reduce_scatter``, ``broadcast``).

Where the reference records an argument and then ignores it, this graph acts on it:
``allreduce(op=)`` is honoured including ``avg`` (runtime.py:211-216 always sums),
``all_to_all(scatter_dim, gather_dim)`` moves the named dimensions (runtime.py:218-226 does a flat
exchange), overlap groups change how the runtimes issue work, and ``execute(stream=)`` runs on
that stream.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional, Sequence

import torch

from .exceptions import (
    AlreadyCompiledError,
    CyclicDependencyError,
    ShapeMismatchError,
    ValidationError,
)
from .nodes import OverlapGroup, TaskNode, TaskType
from .schedule import TaskSchedule
from .validation import (
    validate_dtype_match,
    validate_linear_shapes,
    validate_matmul_shapes,
    validate_same_device,
    validate_tensor,
)

_REDUCE_OPS = ("sum", "avg", "max", "min", "prod")


def _storage_key(t: torch.Tensor):
    if t.numel() == 0:
        return ("id", id(t))
    return ("st", t.device.type, t.device.index, t.untyped_storage().data_ptr())


def _byte_range(t: torch.Tensor):
    start = t.storage_offset() * t.element_size()
    if t.is_contiguous():
        return start, start + t.numel() * t.element_size()
    span = 1
    for size, stride in zip(t.shape, t.stride()):
        span += (size - 1) * abs(stride)
    return start, start + span * t.element_size()


class TaskGraph:
    def __init__(self, num_workers: Optional[int] = None, device: Optional[torch.device] = None):
        self._explicit_device = device is not None
        self.device: torch.device = torch.device(device) if device is not None else self._default_device()
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
        self.num_workers = int(num_workers) if num_workers is not None else self._auto_detect_workers()
        self._nodes: List[TaskNode] = []
        self._overlap_groups: List[OverlapGroup] = []
        self._compiled = False
        self._schedule: Optional[TaskSchedule] = None
        self._runtime = None
        self._next_node_id = 0
        self._weights: Dict[str, torch.Tensor] = {}
        self.runtime_kind: Optional[str] = None
        self._heap_outputs: List[torch.Tensor] = []      # outputs this graph took from the symmetric heap

    # ------------------------------------------------------------------ construction helpers
    @staticmethod
    def _default_device() -> torch.device:
        if torch.cuda.is_available():
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    def _auto_detect_workers(self) -> int:
        if self.device.type == "cuda" and torch.cuda.is_available():
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            return max(1, sms)          # every SM runs a worker CTA; static programs need no scheduler CTA
        return max(1, min(8, os.cpu_count() or 1))

    def _check_not_compiled(self) -> None:
        if self._compiled:
            raise AlreadyCompiledError()

    def _adopt_device(self, t: torch.Tensor) -> None:
        # Without an explicit device the graph follows its first tensor when that does not
        # contradict the default (a CUDA box defaults to CUDA and rejects CPU tensors).
        if not self._explicit_device and not self._nodes and t.device.type == self.device.type:
            self.device = t.device

    def _validate(self, t, name: str, method: str, **kw) -> None:
        validate_tensor(t, name, method, **kw)
        self._adopt_device(t)
        validate_tensor(t, name, method, device=self.device)

    def _add_node(self, node: TaskNode) -> TaskNode:
        node._node_id = self._next_node_id
        self._next_node_id += 1
        if not node.name:
            node.name = f"{node.task_type.name.lower()}_{node._node_id}"
        self._nodes.append(node)
        return node

    def _new(self, ttype: TaskType, name, inputs, outputs, dims=(), **attrs) -> TaskNode:
        return self._add_node(TaskNode(name=name or "", task_type=ttype, inputs=list(inputs),
                                       outputs=list(outputs), dims=list(dims), attrs=dict(attrs)))

    def _out_like(self, ref: torch.Tensor, shape, output: Optional[torch.Tensor], method: str,
                  peer_written: bool = False) -> torch.Tensor:
        shape = tuple(shape)
        if output is None:
            if peer_written and ref.is_cuda:
                # A buffer other ranks write into (all-gather, all-to-all) comes out of the symmetric heap when one
                # exists: peers then push straight into it, where a private tensor would need a heap stand-in
                # of the same size plus a copy inside the launch. Every rank builds the same graph, so the offsets
                # agree.
                from ..comm.process_group import get_world_size
                from ..parallel.symm_heap import current_heap
                heap = current_heap() if get_world_size() > 1 else None
                if heap is not None:
                    try:
                        out = heap.alloc(shape, ref.dtype)
                        self._heap_outputs.append(out)
                        return out
                    except MemoryError:
                        pass
            return torch.empty(shape, dtype=ref.dtype, device=ref.device)
        self._validate(output, "output", method)
        if tuple(output.shape) != shape:
            raise ShapeMismatchError(method, f"output has shape {tuple(output.shape)}, expected {shape}",
                                     "pre-allocate the output with the shape the operation produces")
        validate_dtype_match(ref, "input", output, "output")
        return output

    # ------------------------------------------------------------------ compute nodes
    def linear(self, input, weight, bias=None, name: Optional[str] = None, output=None,
               activation: Optional[str] = None) -> TaskNode:
        """``output = input @ weight.T (+ bias)``; ``weight`` is [out_features, in_features]."""
        self._check_not_compiled()
        self._validate(input, "input", "linear", min_ndim=1)
        self._validate(weight, "weight", "linear", ndim=2)
        if bias is not None:
            self._validate(bias, "bias", "linear", ndim=1)
        validate_linear_shapes(input, weight, bias)
        validate_dtype_match(input, "input", weight, "weight")
        if bias is not None:
            validate_dtype_match(input, "input", bias, "bias")
        validate_same_device([input, weight] + ([bias] if bias is not None else []),
                             ["input", "weight"] + (["bias"] if bias is not None else []))
        if activation not in (None, "gelu", "silu", "swiglu"):
            raise ValidationError(f"unknown activation {activation!r} in linear()\nHint: use None, 'gelu', 'silu' or 'swiglu'")
        n_out = weight.shape[0] // 2 if activation == "swiglu" else weight.shape[0]
        out = self._out_like(input, tuple(input.shape[:-1]) + (n_out,), output, "linear")
        ins = [input, weight] + ([bias] if bias is not None else [])
        return self._new(TaskType.LINEAR, name, ins, [out], [weight.shape[1], weight.shape[0]],
                         has_bias=bias is not None, activation=activation)

    def matmul(self, a, b, name: Optional[str] = None, output=None) -> TaskNode:
        """``output = a @ b`` for 2-D ``a`` [M, K] and ``b`` [K, N]."""
        self._check_not_compiled()
        self._validate(a, "a", "matmul", ndim=2)
        self._validate(b, "b", "matmul", ndim=2)
        validate_matmul_shapes(a, b)
        validate_dtype_match(a, "a", b, "b")
        validate_same_device([a, b], ["a", "b"])
        out = self._out_like(a, (a.shape[0], b.shape[1]), output, "matmul")
        return self._new(TaskType.MATMUL, name, [a, b], [out], [a.shape[0], b.shape[1], a.shape[1]])

    def custom(self, fn: Callable, inputs: Sequence[torch.Tensor], outputs: Sequence[torch.Tensor],
               name: Optional[str] = None, is_comm: bool = False) -> TaskNode:
        """Host-callable escape hatch: ``outputs[0].copy_(fn(*inputs))`` (or in place if ``fn`` returns None)."""
        self._check_not_compiled()
        if not callable(fn):
            raise ValidationError(f"'fn' must be callable in custom(), got {type(fn).__name__}\n"
                                  "Hint: pass a function taking the input tensors and returning the result")
        if inputs is None or outputs is None:
            raise ValidationError("'inputs' and 'outputs' must be sequences of tensors in custom()\nHint: pass lists")
        for i, t in enumerate(inputs):
            self._validate(t, f"inputs[{i}]", "custom")
        for i, t in enumerate(outputs):
            self._validate(t, f"outputs[{i}]", "custom")
        ttype = TaskType.CUSTOM_COMM if is_comm else TaskType.CUSTOM_COMPUTE
        node = self._new(ttype, name, inputs, outputs)
        node.custom_fn = fn
        return node

    def _unary(self, ttype: TaskType, method: str, x, name, output, **attrs) -> TaskNode:
        self._check_not_compiled()
        self._validate(x, "input", method, min_ndim=1)
        out = self._out_like(x, x.shape, output, method)
        return self._new(ttype, name, [x], [out], [x.shape[-1]], **attrs)

    def gelu(self, input, name=None, output=None) -> TaskNode:
        return self._unary(TaskType.GELU, "gelu", input, name, output)

    def silu(self, input, name=None, output=None) -> TaskNode:
        return self._unary(TaskType.SILU, "silu", input, name, output)

    def softmax(self, input, name=None, output=None) -> TaskNode:
        return self._unary(TaskType.SOFTMAX, "softmax", input, name, output)

    def scale(self, input, factor: float, name=None, output=None) -> TaskNode:
        return self._unary(TaskType.SCALE, "scale", input, name, output, factor=float(factor))

    def rmsnorm(self, input, weight, eps: float = 1e-6, name=None, output=None) -> TaskNode:
        self._check_not_compiled()
        self._validate(input, "input", "rmsnorm", min_ndim=1)
        self._validate(weight, "weight", "rmsnorm", ndim=1)
        if weight.shape[0] != input.shape[-1]:
            raise ShapeMismatchError("rmsnorm", f"weight has {weight.shape[0]} elements, input rows have {input.shape[-1]}")
        out = self._out_like(input, input.shape, output, "rmsnorm")
        return self._new(TaskType.RMSNORM, name, [input, weight], [out], [input.shape[-1]], eps=float(eps))

    def layernorm(self, input, weight, bias, eps: float = 1e-5, name=None, output=None) -> TaskNode:
        self._check_not_compiled()
        self._validate(input, "input", "layernorm", min_ndim=1)
        self._validate(weight, "weight", "layernorm", ndim=1)
        self._validate(bias, "bias", "layernorm", ndim=1)
        if weight.shape[0] != input.shape[-1] or bias.shape[0] != input.shape[-1]:
            raise ShapeMismatchError("layernorm", f"weight/bias have {weight.shape[0]}/{bias.shape[0]} elements, "
                                                  f"input rows have {input.shape[-1]}")
        out = self._out_like(input, input.shape, output, "layernorm")
        return self._new(TaskType.LAYERNORM, name, [input, weight, bias], [out], [input.shape[-1]], eps=float(eps))

    def silu_gate(self, gate, up, name=None, output=None) -> TaskNode:
        """``output = silu(gate) * up`` (the SwiGLU gate)."""
        self._check_not_compiled()
        self._validate(gate, "gate", "silu_gate", min_ndim=1)
        self._validate(up, "up", "silu_gate", min_ndim=1)
        if gate.shape != up.shape:
            raise ShapeMismatchError("silu_gate", f"gate {tuple(gate.shape)} vs up {tuple(up.shape)}")
        validate_dtype_match(gate, "gate", up, "up")
        out = self._out_like(gate, gate.shape, output, "silu_gate")
        return self._new(TaskType.SILU_GATE, name, [gate, up], [out], [gate.shape[-1]])

    def add(self, a, b, name=None, output=None) -> TaskNode:
        self._check_not_compiled()
        self._validate(a, "a", "add", min_ndim=1)
        self._validate(b, "b", "add", min_ndim=1)
        if a.shape != b.shape:
            raise ShapeMismatchError("add", f"a {tuple(a.shape)} vs b {tuple(b.shape)}")
        validate_dtype_match(a, "a", b, "b")
        out = self._out_like(a, a.shape, output, "add")
        return self._new(TaskType.ADD, name, [a, b], [out], [a.shape[-1]])

    def rope(self, input, cos, sin, name=None, output=None) -> TaskNode:
        """Rotary embedding (half-rotation form) on ``input`` [tokens, heads, head_dim] with
        ``cos`` / ``sin`` [tokens, head_dim // 2]."""
        self._check_not_compiled()
        self._validate(input, "input", "rope", ndim=3)
        self._validate(cos, "cos", "rope", ndim=2)
        self._validate(sin, "sin", "rope", ndim=2)
        if cos.shape != sin.shape or cos.shape[0] != input.shape[0] or cos.shape[1] * 2 != input.shape[2]:
            raise ShapeMismatchError("rope", f"input {tuple(input.shape)}, cos {tuple(cos.shape)}, sin {tuple(sin.shape)}",
                                     "cos and sin must be [tokens, head_dim // 2]")
        out = self._out_like(input, input.shape, output, "rope")
        return self._new(TaskType.ROPE, name, [input, cos, sin], [out], list(input.shape))

    # ------------------------------------------------------------------ communication nodes
    def allreduce(self, tensor, name: Optional[str] = None, op: str = "sum") -> TaskNode:
        """In-place all-reduce over the default process group; ``task.output is tensor``."""
        self._check_not_compiled()
        self._validate(tensor, "tensor", "allreduce")
        op = str(op).lower()
        if op not in _REDUCE_OPS:
            raise ValidationError(f"unknown reduce op {op!r} in allreduce()\nHint: use one of {_REDUCE_OPS}")
        return self._new(TaskType.ALLREDUCE, name, [tensor], [tensor], [tensor.numel()], op=op)

    def allgather(self, tensor, name: Optional[str] = None, output=None) -> TaskNode:
        """Gathers every rank's ``tensor`` along dim 0 into ``output`` [world * n, ...]."""
        self._check_not_compiled()
        self._validate(tensor, "tensor", "allgather", min_ndim=1)
        from ..comm.process_group import get_world_size
        world = get_world_size()
        out = self._out_like(tensor, (tensor.shape[0] * world,) + tuple(tensor.shape[1:]), output, "allgather",
                             peer_written=True)
        return self._new(TaskType.ALLGATHER, name, [tensor], [out], [tensor.numel()])

    def reduce_scatter(self, tensor, name: Optional[str] = None, output=None, op: str = "sum") -> TaskNode:
        """Reduces ``tensor`` over ranks and leaves dim-0 chunk ``rank`` in ``output``."""
        self._check_not_compiled()
        self._validate(tensor, "tensor", "reduce_scatter", min_ndim=1)
        from ..comm.process_group import get_world_size
        world = get_world_size()
        if tensor.shape[0] % world != 0:
            raise ShapeMismatchError("reduce_scatter", f"dim 0 ({tensor.shape[0]}) is not divisible by world size {world}")
        out = self._out_like(tensor, (tensor.shape[0] // world,) + tuple(tensor.shape[1:]), output, "reduce_scatter")
        return self._new(TaskType.REDUCE_SCATTER, name, [tensor], [out], [tensor.numel()], op=str(op).lower())

    def broadcast(self, tensor, src: int = 0, name: Optional[str] = None) -> TaskNode:
        self._check_not_compiled()
        self._validate(tensor, "tensor", "broadcast")
        return self._new(TaskType.BROADCAST, name, [tensor], [tensor], [tensor.numel()], src=int(src))

    def all_to_all(self, input, name: Optional[str] = None, scatter_dim: int = 2, gather_dim: int = 1,
                   output=None) -> TaskNode:
        """Splits ``scatter_dim`` over ranks and concatenates what arrives along ``gather_dim``
        (the Ulysses head <-> sequence exchange for 4-D [B, S/P, H, D] inputs)."""
        self._check_not_compiled()
        self._validate(input, "input", "all_to_all", min_ndim=1)
        from ..comm.process_group import get_world_size
        world = get_world_size()
        nd = input.dim()
        sd, gd = scatter_dim % nd if nd else 0, gather_dim % nd if nd else 0
        if nd < 2 or sd == gd:
            sd = gd = 0          # flat exchange of equal dim-0 chunks
        shape = list(input.shape)
        if world > 1:
            if shape[sd] % world != 0:
                raise ShapeMismatchError("all_to_all", f"dim {sd} ({shape[sd]}) is not divisible by world size {world}")
            if sd != gd:
                shape[sd] //= world
                shape[gd] *= world
        out = self._out_like(input, shape, output, "all_to_all", peer_written=True)
        return self._new(TaskType.ALL_TO_ALL, name, [input], [out], list(input.shape), scatter_dim=sd, gather_dim=gd)

    # ------------------------------------------------------------------ overlap
    def overlap(self, compute_tasks: Sequence[TaskNode], comm_tasks: Sequence[TaskNode]) -> OverlapGroup:
        self._check_not_compiled()
        group = OverlapGroup(self, list(compute_tasks), list(comm_tasks))
        self._overlap_groups.append(group)
        return group

    # ------------------------------------------------------------------ compile / execute
    def compile(self, runtime: Optional[str] = None) -> "TaskGraph":
        if self._compiled:
            return self
        self._infer_dependencies()
        self._detect_cycles()
        self._assign_events()
        for g in self._overlap_groups:
            if not g._explicit:
                g.auto_waves()
        self._schedule = TaskSchedule(self._nodes, self.num_workers)
        self._init_runtime(runtime)
        self._compiled = True
        return self

    def execute(self, stream=None) -> None:
        if not self._compiled:
            self.compile()
        self._runtime.execute(self._schedule, stream=stream)

    def release(self) -> None:
        """Returns what this graph holds in the symmetric heap (peer-written outputs it allocated itself, and the
        event counters and staging buffers of its persistent program). Collective: every rank calls it at the
        same point; the graph must not run again."""
        from ..parallel.symm_heap import current_heap
        heap = current_heap()
        prog = getattr(self._runtime, "_program", None)
        if heap is None or (not self._heap_outputs and getattr(prog, "heap", None) is None):
            return
        from ..comm.process_group import barrier
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        barrier()
        if prog is not None and getattr(prog, "heap", None) is not None and prog.d_events is not None:
            prog.free_heap()
        for t in self._heap_outputs:
            heap.free(t)
        self._heap_outputs = []
        self._compiled, self._runtime = False, None

    def _infer_dependencies(self) -> None:
        """RAW, WAW and WAR edges from the byte ranges nodes read and write."""
        writers: Dict[object, List] = {}   # storage -> [(lo, hi, node)] last writers
        readers: Dict[object, List] = {}   # storage -> [(lo, hi, node)] readers since the last write

        def overlaps(a_lo, a_hi, b_lo, b_hi):
            return a_lo < b_hi and b_lo < a_hi

        for node in self._nodes:
            for t in node.inputs:
                key = _storage_key(t)
                lo, hi = _byte_range(t)
                for (wlo, whi, w) in writers.get(key, ()):
                    if w is not node and overlaps(lo, hi, wlo, whi):
                        node.add_dependency(w)
            for t in node.outputs:
                key = _storage_key(t)
                lo, hi = _byte_range(t)
                for (wlo, whi, w) in writers.get(key, ()):
                    if w is not node and overlaps(lo, hi, wlo, whi):
                        node.add_dependency(w)
                for (rlo, rhi, r) in readers.get(key, ()):
                    if r is not node and overlaps(lo, hi, rlo, rhi):
                        node.add_dependency(r)
            for t in node.inputs:
                key = _storage_key(t)
                lo, hi = _byte_range(t)
                readers.setdefault(key, []).append((lo, hi, node))
            for t in node.outputs:
                key = _storage_key(t)
                lo, hi = _byte_range(t)
                kept = [(a, b, w) for (a, b, w) in writers.get(key, []) if not (lo <= a and b <= hi)]
                kept.append((lo, hi, node))
                writers[key] = kept
                readers[key] = [(a, b, r) for (a, b, r) in readers.get(key, []) if not overlaps(lo, hi, a, b) or r is node]

    def _detect_cycles(self) -> None:
        WHITE, GREY, BLACK = 0, 1, 2
        colour = {id(n): WHITE for n in self._nodes}
        for root in self._nodes:
            if colour[id(root)] != WHITE:
                continue
            stack = [(root, iter(root.depends_on))]
            path = [root]
            colour[id(root)] = GREY
            while stack:
                node, it = stack[-1]
                advanced = False
                for dep in it:
                    c = colour.get(id(dep), BLACK)
                    if c == GREY:
                        idx = next(i for i, p in enumerate(path) if p is dep)
                        raise CyclicDependencyError([p.name for p in path[idx:]] + [dep.name])
                    if c == WHITE:
                        colour[id(dep)] = GREY
                        stack.append((dep, iter(dep.depends_on)))
                        path.append(dep)
                        advanced = True
                        break
                if not advanced:
                    colour[id(node)] = BLACK
                    stack.pop()
                    path.pop()

    def _assign_events(self) -> None:
        for i, n in enumerate(self._nodes):
            n._event_id = i

    def _init_runtime(self, kind: Optional[str] = None) -> None:
        from ..config import config
        from . import runtime as rt
        kind = kind or os.environ.get("MACO_RUNTIME") or getattr(config, "runtime", "auto")
        if self.device.type != "cuda":
            kind = "reference"
        elif kind == "auto":
            kind = "persistent" if rt.PersistentRuntime.can_run(self) else "stream"
        if kind == "persistent":
            self._runtime = rt.PersistentRuntime(self)
        elif kind == "stream":
            self._runtime = rt.StreamRuntime(self.device, graph=self)
        elif kind == "reference":
            self._runtime = rt.ReferenceRuntime(self.device, graph=self)
        else:
            raise ValidationError(f"unknown runtime {kind!r}\nHint: use 'auto', 'persistent', 'stream' or 'reference'")
        self.runtime_kind = kind

    # ------------------------------------------------------------------ weights / checkpoint
    def register_weight(self, name: str, tensor: torch.Tensor) -> torch.Tensor:
        """Names a tensor so that ``state_dict`` / ``load_state_dict`` can save and restore it."""
        self._weights[name] = tensor
        return tensor

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {k: v.detach().clone() for k, v in self._weights.items()}

    def load_state_dict(self, state: Dict[str, torch.Tensor], strict: bool = True) -> None:
        missing = [k for k in self._weights if k not in state]
        unexpected = [k for k in state if k not in self._weights]
        if strict and (missing or unexpected):
            raise KeyError(f"state_dict mismatch: missing {missing}, unexpected {unexpected}")
        for k, v in state.items():
            if k in self._weights:
                self._weights[k].copy_(v)       # in place: compiled task tables keep their pointers

    # ------------------------------------------------------------------ reporting
    def stats(self) -> dict:
        """Per-task-type timing of the last execute (persistent runtime with tracing on), else {}."""
        if self._runtime is not None and hasattr(self._runtime, "stats"):
            return self._runtime.stats()
        return {}

    def summary(self) -> str:
        n_compute = sum(1 for n in self._nodes if n.is_compute)
        n_comm = sum(1 for n in self._nodes if n.is_comm)
        lines = [
            "TaskGraph Summary",
            f"  Device: {self.device}",
            f"  Workers: {self.num_workers}",
            f"  Total nodes: {len(self._nodes)}",
            f"  Compute nodes: {n_compute}",
            f"  Comm nodes: {n_comm}",
            f"  Overlap groups: {len(self._overlap_groups)}",
            f"  Compiled: {self._compiled}",
        ]
        if self._compiled and self._schedule is not None:
            lines.append(f"  Execution waves: {len(self._schedule.waves)}")
            lines.append(f"  Runtime: {self.runtime_kind}")
            if hasattr(self._runtime, "describe"):
                lines.append(f"  {self._runtime.describe()}")
            for i, wave in enumerate(self._schedule.waves[:16]):
                lines.append(f"    wave {i}: " + ", ".join(n.name for n in wave[:8]) + (" ..." if len(wave) > 8 else ""))
        return "\n".join(lines)

    def __repr__(self) -> str:
        return (f"TaskGraph(nodes={len(self._nodes)}, workers={self.num_workers}, device={self.device}, "
                f"compiled={self._compiled})")

    def __len__(self) -> int:
        return len(self._nodes)
