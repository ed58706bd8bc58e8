"""Collective patterns with one call each: allreduce, allgather, reduce_scatter, send/recv,
all_to_all (list, single, 4-D Ulysses).

API of the reference's maco/comm/patterns.py:12-490. Differences that matter: ``AVG`` really
averages (the reference maps AVG to SUM and never divides, patterns.py:459-461), and when the
active backend is "peer" and the tensor lives in the symmetric heap the call is served by this
package's own in-kernel collectives instead of torch.distributed.
"""
from __future__ import annotations

from enum import Enum
from typing import List, Optional

import torch
import torch.distributed as dist

from ._compat import list_all_to_all
from .process_group import get_rank, get_world_size


class ReduceOp(Enum):
    SUM = "sum"
    PRODUCT = "prod"
    MIN = "min"
    MAX = "max"
    AVG = "avg"


SUM, PRODUCT, MIN, MAX, AVG = ReduceOp.SUM, ReduceOp.PRODUCT, ReduceOp.MIN, ReduceOp.MAX, ReduceOp.AVG


def _norm_op(op) -> ReduceOp:
    if isinstance(op, ReduceOp):
        return op
    if isinstance(op, str):
        return ReduceOp({"product": "prod", "mean": "avg"}.get(op.lower(), op.lower()))
    if op == dist.ReduceOp.SUM:
        return ReduceOp.SUM
    if op == dist.ReduceOp.MAX:
        return ReduceOp.MAX
    if op == dist.ReduceOp.MIN:
        return ReduceOp.MIN
    if op == dist.ReduceOp.PRODUCT:
        return ReduceOp.PRODUCT
    return ReduceOp.SUM


def _convert_op(op):
    """Maps to (torch.distributed op, post-scale). AVG = SUM followed by a divide by world size."""
    op = _norm_op(op)
    table = {ReduceOp.SUM: dist.ReduceOp.SUM, ReduceOp.PRODUCT: dist.ReduceOp.PRODUCT,
             ReduceOp.MIN: dist.ReduceOp.MIN, ReduceOp.MAX: dist.ReduceOp.MAX, ReduceOp.AVG: dist.ReduceOp.SUM}
    return table[op], (1.0 / get_world_size() if op == ReduceOp.AVG else None)


class _AsyncHandle:
    def __init__(self, work=None, tensor=None, post=None):
        self._work, self._tensor, self._post, self._done = work, tensor, post, False

    def wait(self):
        if not self._done:
            if self._work is not None:
                self._work.wait()
            if self._post is not None:
                self._tensor = self._post()
            self._done = True
        return self._tensor

    def is_completed(self) -> bool:
        return self._done or self._work is None or self._work.is_completed()


def _peer_backend_for(*tensors):
    """Returns the peer backend when it is active and owns every given tensor, else None."""
    try:
        from ..parallel import symm_heap
    except Exception:
        return None
    heap = symm_heap.current_heap()
    if heap is None:
        return None
    for t in tensors:
        if not heap.owns(t):
            return None
    return heap


def allreduce(tensor: torch.Tensor, op=ReduceOp.SUM, async_op: bool = False, overlap_with_next: bool = False,
              priority: int = 0, overlap_group=None, group=None):
    """In-place all-reduce. Returns the tensor, or a handle when ``async_op``."""
    if get_world_size() == 1:
        return _AsyncHandle(tensor=tensor) if async_op else tensor
    rop = _norm_op(op)
    heap = _peer_backend_for(tensor) if group is None else None
    if heap is not None and rop in (ReduceOp.SUM, ReduceOp.AVG) and tensor.dtype in (torch.bfloat16, torch.float32):
        from ..parallel import collectives
        collectives.all_reduce(tensor, avg=(rop == ReduceOp.AVG))
        return _AsyncHandle(tensor=tensor) if async_op else tensor
    dop, scale = _convert_op(rop)
    work = dist.all_reduce(tensor, op=dop, group=group, async_op=async_op)
    post = (lambda: tensor.mul_(scale)) if scale is not None else None
    if async_op:
        return _AsyncHandle(work, tensor, post)
    if post is not None:
        post()
    return tensor


def allgather(tensor: torch.Tensor, async_op: bool = False, group=None):
    """Returns ``[world, *tensor.shape]``."""
    world = get_world_size()
    if world == 1:
        out = tensor.unsqueeze(0)
        return _AsyncHandle(tensor=out) if async_op else out
    out = torch.empty((world,) + tuple(tensor.shape), dtype=tensor.dtype, device=tensor.device)
    work = dist.all_gather_into_tensor(out.view(world * tensor.shape[0], *tensor.shape[1:]) if tensor.dim() else out,
                                       tensor.contiguous(), group=group, async_op=async_op)
    return _AsyncHandle(work, out) if async_op else out


def reduce_scatter(tensor: torch.Tensor, op=ReduceOp.SUM, async_op: bool = False, group=None):
    """Reduces over ranks and returns dim-0 chunk ``rank``: ``[N / world, ...]``."""
    world = get_world_size()
    if world == 1:
        return _AsyncHandle(tensor=tensor) if async_op else tensor
    if tensor.shape[0] % world != 0:
        raise ValueError(f"reduce_scatter: dim 0 ({tensor.shape[0]}) not divisible by world size {world}")
    dop, scale = _convert_op(op)
    out = torch.empty((tensor.shape[0] // world,) + tuple(tensor.shape[1:]), dtype=tensor.dtype, device=tensor.device)
    src = tensor.contiguous()
    if dist.get_backend(group) == "gloo":
        # gloo has no reduce_scatter: all-reduce a copy and keep this rank's chunk.
        tmp = src.clone()
        dist.all_reduce(tmp, op=dop, group=group)
        out.copy_(tmp.chunk(world, dim=0)[get_rank()])
        work = None
    else:
        work = dist.reduce_scatter_tensor(out, src, op=dop, group=group, async_op=async_op)
    post = (lambda: out.mul_(scale)) if scale is not None else None
    if async_op:
        return _AsyncHandle(work, out, post)
    if post is not None:
        post()
    return out


def send(tensor: torch.Tensor, dst: int, tag: int = 0, async_op: bool = False, group=None):
    if get_world_size() == 1:
        return None
    if async_op:
        return _AsyncHandle(dist.isend(tensor, dst=dst, tag=tag, group=group), tensor)
    dist.send(tensor, dst=dst, tag=tag, group=group)
    return None


def recv(tensor: torch.Tensor, src: int, tag: int = 0, async_op: bool = False, group=None):
    if get_world_size() == 1:
        return tensor
    if async_op:
        return _AsyncHandle(dist.irecv(tensor, src=src, tag=tag, group=group), tensor)
    dist.recv(tensor, src=src, tag=tag, group=group)
    return tensor


def all_to_all(tensor: torch.Tensor, scatter_dim: int = 0, gather_dim: int = 0, async_op: bool = False, group=None):
    world = get_world_size()
    if world == 1:
        return _AsyncHandle(tensor=tensor) if async_op else tensor
    send_list = [c.contiguous() for c in torch.tensor_split(tensor, world, dim=scatter_dim)]
    recv_list = [torch.empty_like(c) for c in send_list]
    work = list_all_to_all(recv_list, send_list, group=group, async_op=async_op)
    fin = lambda: torch.cat(recv_list, dim=gather_dim)
    if async_op:
        return _AsyncHandle(work, None, fin)
    return fin()


def all_to_all_single(output: Optional[torch.Tensor], input: torch.Tensor,
                      output_split_sizes: Optional[List[int]] = None, input_split_sizes: Optional[List[int]] = None,
                      async_op: bool = False, group=None):
    if output is None:
        output = torch.empty_like(input)
    if get_world_size() == 1:
        output.copy_(input)
        return _AsyncHandle(tensor=output) if async_op else output
    if dist.get_backend(group) == "gloo" and (output_split_sizes or input_split_sizes):
        ins = list(input.split(input_split_sizes or input.shape[0] // get_world_size(), dim=0))
        outs = list(output.split(output_split_sizes or output.shape[0] // get_world_size(), dim=0))
        outs_c = [torch.empty_like(o) for o in outs]
        list_all_to_all(outs_c, [i.contiguous() for i in ins], group=group)
        for o, c in zip(outs, outs_c):
            o.copy_(c)
        return _AsyncHandle(tensor=output) if async_op else output
    work = dist.all_to_all_single(output, input.contiguous(), output_split_sizes, input_split_sizes,
                                  group=group, async_op=async_op)
    return _AsyncHandle(work, output) if async_op else output


def all_to_all_4D(tensor: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1, async_op: bool = False, group=None,
                  out: Optional[torch.Tensor] = None):
    """Ulysses layout switch. (scatter 2, gather 1): [B, S/P, H, D] -> [B, S, H/P, D];
    (scatter 1, gather 2): [B, S, H/P, D] -> [B, S/P, H, D]. One exchange of a single buffer.
    With the peer backend and a tensor in the symmetric heap the exchange runs inside this package's
    kernel; the result is written into ``out`` (a heap tensor) when given, and is otherwise a fresh tensor
    (a copy out of the kernel's receive buffer), so successive calls never alias."""
    if tensor.dim() != 4:
        raise ValueError(f"all_to_all_4D expects a 4-D tensor, got {tensor.dim()}-D")
    world = get_world_size()
    if world == 1:
        return _AsyncHandle(tensor=tensor) if async_op else tensor
    heap = _peer_backend_for(tensor) if group is None else None
    if heap is not None and tensor.dtype in (torch.bfloat16, torch.float16, torch.float32):
        from ..parallel import collectives
        if out is not None:
            res = collectives.all_to_all_4d(tensor, scatter_dim, gather_dim, out=out)
        else:
            res = collectives.all_to_all_4d(tensor, scatter_dim, gather_dim).clone()
        return _AsyncHandle(tensor=res) if async_op else res
    P = world
    if (scatter_dim, gather_dim) == (2, 1):
        B, s, H, D = tensor.shape
        if H % P:
            raise ValueError(f"heads ({H}) not divisible by world size {P}")
        send = tensor.reshape(B, s, P, H // P, D).permute(2, 0, 1, 3, 4).contiguous()   # [P, B, s, h, D]
        recv = torch.empty_like(send)
        work = dist.all_to_all_single(recv, send, group=group, async_op=async_op)
        fin = lambda: recv.permute(1, 0, 2, 3, 4).reshape(B, P * s, H // P, D)
    elif (scatter_dim, gather_dim) == (1, 2):
        B, S, h, D = tensor.shape
        if S % P:
            raise ValueError(f"sequence ({S}) not divisible by world size {P}")
        send = tensor.reshape(B, P, S // P, h, D).permute(1, 0, 2, 3, 4).contiguous()   # [P, B, s, h, D]
        recv = torch.empty_like(send)
        work = dist.all_to_all_single(recv, send, group=group, async_op=async_op)
        fin = lambda: recv.permute(1, 2, 0, 3, 4).reshape(B, S // P, P * h, D)
    else:
        return all_to_all(tensor, scatter_dim, gather_dim, async_op=async_op, group=group)
    if async_op:
        return _AsyncHandle(work, None, fin)
    return fin()
