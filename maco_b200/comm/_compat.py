"""Backend gaps papered over in one place: gloo has no list all_to_all and no reduce_scatter."""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist


class _DoneWork:
    def wait(self):
        return True

    def is_completed(self) -> bool:
        return True


def list_all_to_all(recv: List[torch.Tensor], send: List[torch.Tensor], group=None, async_op: bool = False):
    """``dist.all_to_all`` that also works on gloo (point-to-point exchange there)."""
    if dist.get_backend(group) != "gloo":
        return dist.all_to_all(recv, send, group=group, async_op=async_op)
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    recv[rank].copy_(send[rank])
    reqs = []
    for peer in range(world):
        if peer == rank:
            continue
        reqs.append(dist.isend(send[peer], dst=dist.get_global_rank(group, peer) if group is not None else peer, group=group))
        reqs.append(dist.irecv(recv[peer], src=dist.get_global_rank(group, peer) if group is not None else peer, group=group))
    for r in reqs:
        r.wait()
    return _DoneWork()
