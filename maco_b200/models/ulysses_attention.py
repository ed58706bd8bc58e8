"""Ulysses sequence-parallel attention on this package's kernels.

    x [B, S/P, hidden]  (this rank's slice of the sequence)
    q, k, v = x Wq^T, x Wk^T, x Wv^T           [B, S/P, H, D]     tcgen05 GEMM tiles
    all-to-all (scatter heads, gather sequence)  [B, S, H/P, D]     peer pushes straight into the new layout
    attention over the FULL sequence on H/P heads
    all-to-all back                              [B, S/P, H, D]
    out = o Wo^T                                 [B, S/P, hidden]

Two task graphs, each ONE launch of the persistent kernel per rank: (projections + three exchanges) and (inverse
exchange + output projection). Inside a launch an exchange task starts as soon as the GEMM tiles that produce its
tensor are done, while the tiles of the next projection still run; nothing is packed or unpacked (each
(batch, position, destination) slice is one row of a strided push). The attention itself between the two launches
is PyTorch's scaled_dot_product_attention: a prefill attention task is not part of this package yet.

The reference's counterpart (examples/test_overlap_attention.py:78-125) runs cuBLAS projections, three
chunk / contiguous / NCCL all_to_all / cat exchanges on a side stream, and a naive softmax(QK^T)V.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..task_graph.graph import TaskGraph


class UlyssesAttention:
    def __init__(self, batch: int, seq_len: int, heads: int, head_dim: int, hidden: int, *, rank: int = 0, world: int = 1,
                 heap=None, dtype: torch.dtype = torch.bfloat16, seed: int = 0, weight_std: float = 0.05,
                 device: Optional[torch.device] = None):
        if seq_len % world or heads % world:
            raise ValueError("sequence length and heads must be divisible by the world size")
        if world > 1 and heap is None:
            raise ValueError("world > 1 needs the symmetric heap")
        self.B, self.S, self.H, self.D, self.hidden = batch, seq_len, heads, head_dim, hidden
        self.rank, self.world, self.dtype = rank, world, dtype
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        s, hp = seq_len // world, heads // world
        g = torch.Generator(device="cpu").manual_seed(seed)          # the same weights on every rank
        mk = lambda *shape: (torch.randn(*shape, generator=g) * weight_std).to(dtype).to(dev)
        self.wq, self.wk, self.wv = mk(heads * head_dim, hidden), mk(heads * head_dim, hidden), mk(heads * head_dim, hidden)
        self.wo = mk(hidden, heads * head_dim)
        alloc = (lambda shape: heap.alloc(shape, dtype)) if heap is not None else (lambda shape: torch.empty(shape, device=dev, dtype=dtype))
        self.x = torch.empty(batch * s, hidden, device=dev, dtype=dtype)
        # buffers other ranks write into live in the heap (no stand-in copies inside the launch)
        self.qkv_local = [alloc((batch, s, heads, head_dim)) for _ in range(3)]
        self.qkv_full = [alloc((batch, seq_len, hp, head_dim)) for _ in range(3)]
        self.o_full = alloc((batch, seq_len, hp, head_dim))
        self.o_local = alloc((batch, s, heads, head_dim))
        self.out = torch.empty(batch * s, hidden, device=dev, dtype=dtype)
        g1 = TaskGraph(device=dev)
        for w, loc, full in zip((self.wq, self.wk, self.wv), self.qkv_local, self.qkv_full):
            proj = g1.linear(self.x, w, output=loc.view(batch * s, heads * head_dim))
            g1.all_to_all(loc, scatter_dim=2, gather_dim=1, output=full).add_dependency(proj)
        g1.compile()
        g2 = TaskGraph(device=dev)
        back = g2.all_to_all(self.o_full, scatter_dim=1, gather_dim=2, output=self.o_local)
        g2.linear(self.o_local.view(batch * s, heads * head_dim), self.wo, output=self.out).add_dependency(back)
        g2.compile()
        self.graph_in, self.graph_out = g1, g2

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` [B, S/P, hidden] -> [B, S/P, hidden] for this rank's slice of the sequence."""
        self.x.copy_(x.reshape(self.x.shape))
        self.graph_in.execute()
        q, k, v = (t.transpose(1, 2) for t in self.qkv_full)                    # [B, H/P, S, D]
        o = torch.nn.functional.scaled_dot_product_attention(q, k, v)
        self.o_full.copy_(o.transpose(1, 2))
        self.graph_out.execute()
        return self.out.view(self.B, self.S // self.world, self.hidden)

    __call__ = forward

    def reference(self, x_full: torch.Tensor) -> torch.Tensor:
        """fp32 PyTorch attention over the whole sequence and all heads; returns this rank's rows."""
        B, S, H, D = self.B, self.S, self.H, self.D
        xf = x_full.float().reshape(B * S, self.hidden)
        r = lambda w: (xf @ w.float().t()).to(self.dtype).float().view(B, S, H, D).transpose(1, 2)
        q, k, v = r(self.wq), r(self.wk), r(self.wv)
        o = torch.softmax(q @ k.transpose(-1, -2) * D ** -0.5, -1) @ v           # [B, H, S, D]
        o = o.transpose(1, 2).reshape(B * S, H * D).to(self.dtype).float()
        y = (o @ self.wo.float().t()).view(B, S, self.hidden)
        s = S // self.world
        return y[:, self.rank * s:(self.rank + 1) * s]
