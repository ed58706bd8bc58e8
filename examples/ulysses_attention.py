#!/usr/bin/env python
"""Ulysses sequence parallelism: [B, S/P, H, D] -> all-to-all -> attention over the full sequence on
H/P heads -> inverse all-to-all, with the exchange overlapped against independent compute.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/ulysses_attention.py
(counterpart of the reference's examples/test_overlap_attention.py)"""
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
    B, S, H, D = 2, 512, 8, 64
    s = S // world
    torch.manual_seed(rank)
    q, k, v = (torch.randn(B, s, H, D, device=dev) for _ in range(3))
    w = torch.randn(1024, 1024, device=dev)

    def exchange():
        return [patterns.all_to_all_4D(t, 2, 1) for t in (q, k, v)]      # -> [B, S, H/P, D]

    (qf, kf, vf), side = maco.overlap_all_to_all_with_compute(exchange, lambda: w @ w)
    att = torch.nn.functional.scaled_dot_product_attention(qf.transpose(1, 2), kf.transpose(1, 2), vf.transpose(1, 2))
    out = patterns.all_to_all_4D(att.transpose(1, 2).contiguous(), 1, 2)  # back to [B, S/P, H, D]
    print(f"[rank {rank}] output {tuple(out.shape)}, side compute {tuple(side.shape)}")
    maco.cleanup()


if __name__ == "__main__":
    main()
