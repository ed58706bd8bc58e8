#!/usr/bin/env python
"""Ulysses sequence parallelism on this package's kernels: projections, the three head <-> sequence exchanges and
the inverse exchange + output projection run as two launches of the persistent kernel per rank; the tensors live in
the symmetric heap, so the exchanges are in-kernel peer pushes, not NCCL calls.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/ulysses_attention.py
(counterpart of the reference's examples/test_overlap_attention.py)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist

import maco_b200 as maco
from maco_b200.models.ulysses_attention import UlyssesAttention
from maco_b200.parallel import symm_heap


def main():
    maco.config.set(comm_buffer_size="256MB", backend="peer")
    maco.init(backend="nccl")
    rank, world = maco.get_rank(), maco.get_world_size()
    B, S, H, D, hidden = 2, 1024, 8 * world, 64, 1024
    layer = UlyssesAttention(B, S, H, D, hidden, rank=rank, world=world, heap=symm_heap.current_heap())
    torch.manual_seed(0)
    x_full = torch.randn(B, S, hidden, device="cuda", dtype=torch.bfloat16)
    s = S // world
    out = layer(x_full[:, rank * s:(rank + 1) * s])
    torch.cuda.synchronize()
    ref = layer.reference(x_full)
    err = (out.float() - ref).abs().max().item()
    print(f"[rank {rank}] runtimes {layer.graph_in.runtime_kind}/{layer.graph_out.runtime_kind}, output {tuple(out.shape)}, "
          f"max abs error vs fp32 {err:.3e}")
    if world > 1:
        dist.barrier()
    maco.cleanup()


if __name__ == "__main__":
    main()
