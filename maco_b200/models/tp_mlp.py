"""Tensor-parallel SwiGLU MLP forward with sequence-parallel input and output.

    x_shard [T/P, H]  --all-gather-->  x [T, H]
    h = silu(x Wg^T) * (x Wu^T)        column-parallel gate/up  [H -> F/P each]
    y_shard = reduce_scatter(h Wd^T)   row-parallel down        [F/P -> H]

The whole layer is ONE launch of the persistent kernel per rank. The all-gather is pushed in
128-row chunks by a few communication workers and each gate/up tile waits only for the 128 rows it reads; SwiGLU is applied in the
GEMM epilogue (gate and up weights are interleaved per 256-column tile); the down-projection
epilogue stores every partial tile into the staging slot of the rank that owns those rows, and
that rank sums the slots as their per-block counters fill (with two ranks the own tiles add the
peer's slot in their epilogue and write final rows). With one rank the collectives vanish and the
same two fused GEMMs run.

The reference expresses this layer as separate torch.mm launches plus NCCL calls
(maco/task_graph/runtime.py:188-234, maco/comm/patterns.py:80-175) and its own tensor-parallel
example all-reduces a column-parallel output (examples/tensor_parallel.py:55-61).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import interleave_gate_up
from ..ops.megakernel import BM, ProgramBuilder
from ..parallel import fused


class TPSwiGLUMLP:
    def __init__(self, tokens: int, hidden: int, ffn: int, *, rank: int = 0, world: int = 1, heap=None,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16, seed: int = 0,
                 mode: str = "static", trace: bool = False, weight_std: float = 0.02, num_workers: Optional[int] = None,
                 comm_workers: Optional[int] = None, cta_pair: bool = True, nvls_allgather: bool = False,
                 input_slots: int = 1):
        if tokens % (world * BM) or ffn % (world * 128):
            raise ValueError("tokens must be a multiple of world*128 and ffn of world*128")
        if world > 1 and heap is None:
            raise ValueError("world > 1 needs the symmetric heap")
        self.tokens, self.hidden, self.ffn = tokens, hidden, ffn
        self.rank, self.world, self.heap = rank, world, heap
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dtype = dtype
        self.rows_local = tokens // world
        f_local = ffn // world
        g = torch.Generator(device="cpu").manual_seed(seed * 1000 + rank)
        mk = lambda *s: (torch.randn(*s, generator=g) * weight_std).to(dtype).to(self.device)
        self.w_gate, self.w_up, self.w_down = mk(f_local, hidden), mk(f_local, hidden), mk(hidden, f_local)
        self.w_gate_up = interleave_gate_up(self.w_gate, self.w_up)
        dev = self.device
        if comm_workers is None:
            # one SM pushes roughly 25-30 GB/s into a peer; the shard has to reach world-1 peers before
            # they run out of local rows to work on
            # (8 GPUs, this layer: 12 workers 493 us, 16 workers 459-482 us, 24 workers 479 us)
            comm_workers = 6 if world <= 2 else 16
        # two-CTA GEMM tiles: 256 x 256 per CTA pair (static queues only)
        cta_pair = cta_pair and mode == "static"
        self.h = torch.empty(tokens, f_local, device=dev, dtype=dtype)
        self.y_shard = torch.empty(self.rows_local if world > 1 else tokens, hidden, device=dev, dtype=dtype)
        # ``input_slots`` = 2 builds the program twice over two input buffers (weights, h and the output are shared):
        # an end-to-end loop copies the next input from the host straight into the slot the running launch does not read
        self.programs, self.x_shards = [], []
        for _ in range(max(1, int(input_slots))):
            b = ProgramBuilder(dev, num_workers=num_workers, mode=mode, heap=heap, trace=trace,
                               num_comm_workers=(comm_workers if world > 1 else 0), cta_pair=cta_pair)
            if world == 1:
                x_shard = torch.empty(tokens, hidden, device=dev, dtype=dtype)
                e1 = b.gemm(x_shard, self.w_gate_up, self.h, epilogue="swiglu")
                b.gemm(self.h, self.w_down, self.y_shard, a_ready=e1)
            else:
                # every slot has its own gathered buffer and staging slots: what a peer's launch on one slot writes
                # is never touched by a launch on the other slot, so each program's own fence is all the ordering needed
                x_full = heap.alloc((tokens, hidden), dtype)
                # the input shard IS this rank's slice of the gathered buffer: nothing to copy locally
                x_shard = x_full[rank * self.rows_local:(rank + 1) * self.rows_local]
                staging = heap.alloc((world, self.rows_local, hidden), dtype)
                self.x_full, self.staging = x_full, staging
                fence = fused.epoch_fence_event(b)
                use_mc = nvls_allgather and bool(heap.multicast_base())
                eg = fused.allgather_push(b, x_shard, x_full, fence=fence, multicast=use_mc)
                order = fused.gathered_order(rank, world, self.rows_local // BM, use_mc)
                e1 = b.gemm(x_full, self.w_gate_up, self.h, epilogue="swiglu", a_ready=eg, m_blocks=order)
                _, eo = fused.gemm_reduce_scatter(b, self.h, self.w_down, staging, self.y_shard, a_ready=e1)
                fused.epoch_fence_signal(b, [(eo.all_event[0], eo.all_event[1], False, False),
                                             (e1.all_event[0], e1.all_event[1], False, False)])
            # (a CPU device plans only: the task lists stay in ``self.builders`` for host-side schedule checks)
            self.builders = getattr(self, "builders", []) + [b]
            self.programs.append(b.build() if dev.type == "cuda" else None)
            self.x_shards.append(x_shard)
        self.program, self.x_shard = self.programs[0], self.x_shards[0]

    def forward(self, x_shard: Optional[torch.Tensor] = None, stream=None, slot: int = 0) -> torch.Tensor:
        """Runs the layer on ``x_shard`` [T/P, H] (copied into the layer's input buffer; pass None
        when the caller already wrote ``self.x_shards[slot]``). Returns this rank's output rows."""
        if x_shard is not None:
            self.x_shards[slot].copy_(x_shard, non_blocking=True)
        self.programs[slot].run(stream=stream)
        return self.y_shard

    __call__ = forward

    def reference(self, x_full: torch.Tensor) -> torch.Tensor:
        """fp32 PyTorch result of this rank's PARTIAL product (before the cross-rank sum)."""
        F = torch.nn.functional
        xf = x_full.float()
        h = (F.silu(xf @ self.w_gate.float().t()) * (xf @ self.w_up.float().t())).to(self.dtype).float()
        return h @ self.w_down.float().t()

    def flops(self) -> float:
        """Per-rank FLOPs of one forward."""
        return 2.0 * self.tokens * self.hidden * (self.ffn // self.world) * 3
