"""Data-parallel backward of an MLP stack with the gradient all-reduce overlapped tile by tile.

Model: L layers of ``a_l = gelu(a_{l-1} W_l^T)`` and an MSE loss to a target. One launch of the
persistent kernel per rank runs the whole backward pass:

* ``dZ_{l-1} = (dZ_l W_l) * gelu'(z_{l-1})``  dgrad GEMM with the GELU derivative in the epilogue;
  a tile of layer l-1 starts as soon as the 128 rows it reads of layer l are complete, so the
  dgrad chain is pipelined across layers.
* ``dW_l = dZ_l^T a_{l-1}``  wgrad GEMM (both operands read transposed straight from memory, fp32
  output, the 1/world of the average folded into the epilogue).
* every finished 128-row block of ``dW_l`` is announced to the rank that owns it; that rank's
  communication workers pull the block from all ranks over NVLink, sum in fp32 and write the
  result back to every rank - while the compute workers are already on the next layers.

The reference models this as "matmul on one stream, NCCL all-reduce on another"
(examples/test_real_overlap.py:48-71, benchmarks/benchmark_overlap.py:51-89) with no averaging
(maco/comm/patterns.py:459-461).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import _native as N
from .. import ops
from ..ops.megakernel import BM, COMM_REDUCE_LOCAL_BCAST, ProgramBuilder, _pack_comm
from ..parallel import fused
from ..task_graph.nodes import TaskType


class DPMLPStackBackward:
    def __init__(self, layers: int = 16, hidden: int = 4096, tokens: int = 8192, *, rank: int = 0, world: int = 1,
                 heap=None, device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16, seed: int = 0,
                 mode: str = "static", trace: bool = False, comm_workers: Optional[int] = None, weight_std: float = 0.02,
                 cta_pair: bool = False):
        # two-CTA tiles measured slower here (8.5 ms against 8.0 ms on one GPU: both operands of the wgrad tiles are
        # MN-major, 64-column TMA boxes), so the one-CTA form is the default
        self.cta_pair = cta_pair and mode == "static"
        if tokens % BM or hidden % 256:
            raise ValueError("tokens must be a multiple of 128 and hidden of 256")
        if world > 1 and heap is None:
            raise ValueError("world > 1 needs the symmetric heap")
        self.layers, self.hidden, self.tokens = layers, hidden, tokens
        self.rank, self.world, self.heap, self.dtype = rank, world, heap, dtype
        dev = self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        gw = torch.Generator(device="cpu").manual_seed(seed)                   # weights identical on every rank
        self.weights = [(torch.randn(hidden, hidden, generator=gw) * weight_std).to(dtype).to(dev) for _ in range(layers)]
        gx = torch.Generator(device="cpu").manual_seed(seed * 7919 + 13 + rank)  # data differs per rank
        self.x = torch.randn(tokens, hidden, generator=gx).to(dtype).to(dev)
        self.target = torch.randn(tokens, hidden, generator=gx).to(dtype).to(dev)
        self.z = [torch.empty(tokens, hidden, device=dev, dtype=dtype) for _ in range(layers)]
        self.a = [torch.empty(tokens, hidden, device=dev, dtype=dtype) for _ in range(layers)]
        self.dz = [torch.empty(tokens, hidden, device=dev, dtype=dtype) for _ in range(2)]   # ping-pong
        self.da = torch.empty(tokens, hidden, device=dev, dtype=dtype)
        if world > 1:
            if (hidden // BM) % world:
                raise ValueError("hidden / 128 must be a multiple of world")
            self.dw = heap.alloc((layers, hidden, hidden), torch.float32)
            # staging[l][source rank] holds the partial gradient blocks this rank owns (block mb is owned by rank
            # mb % world and sits at index mb // world); the wgrad epilogues of every rank store into it
            self.staging = heap.alloc((layers, world, hidden // world, hidden), torch.float32)
        else:
            self.dw = torch.empty(layers, hidden, hidden, device=dev, dtype=torch.float32)
        if comm_workers is None:
            # the gradient traffic per rank grows with (world-1)/world; a communication worker moves 25-40 GB/s
            comm_workers = 12
        self._build(mode, trace, comm_workers if world > 1 else 0)

    # ------------------------------------------------------------------ forward (set-up, separate launches)
    def forward(self) -> torch.Tensor:
        cur = self.x
        for l in range(self.layers):
            ops.gemm(cur, self.weights[l], out=self.z[l])
            ops.gelu(self.z[l], out=self.a[l])
            cur = self.a[l]
        return cur

    # ------------------------------------------------------------------ backward program
    def _build(self, mode: str, trace: bool, comm_workers: int) -> None:
        L, H, T, world, rank = self.layers, self.hidden, self.tokens, self.world, self.rank
        b = ProgramBuilder(self.device, mode=mode, heap=self.heap, trace=trace, num_comm_workers=comm_workers,
                           cta_pair=self.cta_pair)
        numel = float(T * H)
        e_da = b.elementwise(int(TaskType.AXPBY), self.a[L - 1], self.da, in1=self.target, rows=T, cols=H,
                             f0=2.0 / numel, f1=-2.0 / numel)
        e_dz = b.elementwise(int(TaskType.GELU_BWD), self.da, self.dz[(L - 1) & 1], in1=self.z[L - 1], rows=T, cols=H,
                             in_ready=[e_da])
        n_blocks = H // BM
        n_tiles_w = (H + 255) // 256
        done_events: List[tuple] = []
        row_bytes = H * 4
        split = 4
        prev_readers = None          # tasks that still read the ping-pong buffer about to be overwritten
        for l in range(L - 1, -1, -1):
            dz_l = self.dz[l & 1]
            inp = self.a[l - 1] if l > 0 else self.x
            e_next = None
            if l > 0:
                # dgrad first: it is the critical path. Overwrites the other ping-pong buffer, which the
                # wgrad of layer l+1 may still be reading: order it behind that wgrad.
                extra = [prev_readers] if prev_readers is not None else []
                e_next = b.gemm(dz_l, self.weights[l], self.dz[(l - 1) & 1], trans_b=True, epilogue="gelu_bwd",
                                aux=self.z[l - 1], a_ready=e_dz, bn=256, extra_waits=extra)
            ready = [b.new_event() for _ in range(n_blocks)] if world > 1 else None
            if world > 1:
                st_off = self.heap.offset_of(self.staging[l])
                slot_bytes = (H // world) * row_bytes

            def per_tile(mb, nb, ready=ready, l=l):
                if ready is None:
                    return {}
                # the tile goes into slot `rank` of the block's owner (a peer store from the epilogue, or a local
                # one when this rank owns the block) at the owner's index of the block
                return dict(peer=mb % world, out_off=st_off + rank * slot_bytes, row_off=(mb // world - mb) * BM,
                            signal_peer=mb % world, signal_peer_event=ready[mb])

            e_w = b.gemm(dz_l, inp, self.dw[l], trans_a=True, trans_b=True, epilogue="f32", alpha=1.0 / world, bn=256,
                         extra_waits=[(e_dz.all_event[0], e_dz.all_event[1], False, False)], per_tile=per_tile)
            prev_readers = (e_w.all_event[0], e_w.all_event[1], False, False)
            if world > 1:
                off = self.heap.offset_of(self.dw[l])
                done = b.new_event()
                n_done = 0
                for mb in range(n_blocks):
                    n_done += split
                    if mb % world != rank:
                        continue
                    for s in range(split):
                        r_own = (mb // world) * BM + s * (BM // split)       # row inside my slots
                        r_glob = mb * BM + s * (BM // split)                 # row of the gradient
                        # sum the `world` local slots (no remote reads: the peers' partials were stored here by
                        # their epilogues) and send the averaged rows to every rank's gradient buffer
                        raw = _pack_comm(st_off + r_own * row_bytes, off + r_glob * row_bytes, row_bytes, row_bytes, row_bytes,
                                         BM // split, N.DTYPE_CODE[torch.float32], -1, COMM_REDUCE_LOCAL_BCAST,
                                         nslots=world, slot_stride=slot_bytes, scale=1.0)
                        b.add_task(int(TaskType.ALLREDUCE), raw, waits=[(ready[mb], world * n_tiles_w, True, False)],
                                   signal_peer=-2, signal_peer_event=done, comm_worker=True)
                done_events.append((done, n_done, True, False))
            else:
                done_events.append((e_w.all_event[0], e_w.all_event[1], False, False))
            if e_next is not None:
                e_dz = e_next
        b.add_task(int(TaskType.NOP), b"", waits=b.join(done_events))
        # (a CPU device plans only: the task list stays in ``self.builder`` for host-side schedule checks)
        self.builder = b
        self.program = b.build() if self.device.type == "cuda" else None

    def backward(self, stream=None) -> torch.Tensor:
        """One persistent launch: all dgrad / wgrad GEMMs plus the averaged gradient all-reduce."""
        self.program.run(stream=stream)
        return self.dw

    def flops(self) -> float:
        return 2.0 * self.tokens * self.hidden * self.hidden * (2 * self.layers - 1)

    # ------------------------------------------------------------------ oracle
    def reference_grads(self) -> torch.Tensor:
        """fp32 autograd gradients of this rank's loss (before averaging over ranks)."""
        ws = [w.float().clone().requires_grad_(True) for w in self.weights]
        cur = self.x.float()
        for w in ws:
            cur = torch.nn.functional.gelu(cur @ w.t(), approximate="tanh")
        loss = torch.nn.functional.mse_loss(cur, self.target.float())
        loss.backward()
        return torch.stack([w.grad for w in ws])
