#!/usr/bin/env python
"""Tensor-parallel SwiGLU MLP with sequence-parallel input/output: all-gather -> GEMM and
GEMM -> reduce-scatter fused into one persistent launch per rank.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/tensor_parallel.py
(the reference's examples/tensor_parallel.py all-reduces a column-parallel output; this is the
column-parallel -> row-parallel pairing with the collectives issued from inside the kernel)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist

import maco_b200 as maco
from maco_b200.models.tp_mlp import TPSwiGLUMLP
from maco_b200.parallel import symm_heap


def main():
    maco.config.set(comm_buffer_size="256MB")
    maco.init(backend="nccl")
    rank, world = maco.get_rank(), maco.get_world_size()
    tokens, hidden, ffn = 2048, 2048, 4096
    layer = TPSwiGLUMLP(tokens, hidden, ffn, rank=rank, world=world, heap=symm_heap.current_heap())
    torch.manual_seed(0)
    x_full = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    rows = tokens // world
    y = layer(x_full[rank * rows:(rank + 1) * rows])
    torch.cuda.synchronize()
    ref = layer.reference(x_full)
    if world > 1:
        dist.all_reduce(ref)
    err = (y.float() - ref[rank * rows:(rank + 1) * rows]).abs().max().item()
    print(f"[rank {rank}] {layer.program.describe()}  max abs err {err:.3e}")
    maco.cleanup()


if __name__ == "__main__":
    main()
