#!/usr/bin/env python
"""All-reduce three ways: library (NCCL / gloo), the peer-memory kernel, and a graph node.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/simple_allreduce.py
(counterpart of the reference's examples/simple_allreduce.py)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import maco_b200 as maco
from maco_b200.comm import patterns


def main():
    cuda = torch.cuda.is_available()
    maco.init(backend="nccl" if cuda else "gloo")
    rank, world = maco.get_rank(), maco.get_world_size()
    dev = maco.ProcessGroupManager().device
    t = torch.full((1 << 20,), float(rank + 1), device=dev)
    patterns.allreduce(t)                                        # torch.distributed
    expect = world * (world + 1) / 2
    print(f"[rank {rank}] library all-reduce ok: {bool(torch.all(t == expect))}")
    if cuda and world > 1:
        from maco_b200.parallel import symm_heap
        heap = symm_heap.current_heap()
        h = heap.alloc((1 << 20,), torch.float32)
        h.fill_(float(rank + 1))
        patterns.allreduce(h, op=patterns.AVG)                   # served by the in-kernel collective
        torch.cuda.synchronize()
        print(f"[rank {rank}] peer-memory all-reduce (avg) ok: {bool(torch.allclose(h, torch.full_like(h, expect / world)))}")
    g = maco.TaskGraph(device=dev)
    u = torch.full((4096,), float(rank), device=dev)
    g.allreduce(u, op="sum")
    g.execute()
    print(f"[rank {rank}] graph all-reduce ok: {bool(torch.all(u == sum(range(world))))}")
    maco.cleanup()


if __name__ == "__main__":
    main()
