"""Expert-parallel mixture-of-experts layer (softmax top-k routing, SwiGLU experts) in one launch.

Per rank, inside the persistent kernel:

1. router GEMM (tcgen05): ``logits = x Wr^T``
2. TOPK tasks: per token the top-k experts and their renormalised softmax weights; a slot in the
   chosen expert's receive slab is taken with an atomic counter and the token row goes, by one bulk
   copy per expert, straight into that slab on the GPU that owns the expert (dispatch all-to-all
   fused with the router permute), with a {token, k, weight} record beside it
3. the per-expert counts are published to the expert owners
4. grouped expert GEMMs over the slabs: gate/up with SwiGLU in the epilogue, then down; tiles whose
   128-row block holds no tokens are skipped by all roles of the worker (run-time counted tiles)
5. the down projection's epilogue scales every valid output row by its routing weight and sends it back into the
   source rank's combine buffer at [token, k] (combine all-to-all fused into the GEMM; ``fused_return=False``: separate
   MOE_RETURN tasks do it from a slab of outputs)
6. the source sums the k rows of every token.

Receive slabs have a fixed capacity per (source rank, expert); routed pairs that do not fit are
dropped for that expert (zero contribution) and counted: the count of every step reaches the host without a
blocking read, and the next ``forward()`` warns or raises (``on_drop``) when it is not zero; ``dropped()`` returns it.

The reference simulates expert parallelism with equal splits on one GPU and a dummy all_to_all node
(examples/benchmark_all_to_all.py:31-127): no router, no top-k, no permute, no variable splits.
"""
from __future__ import annotations

import ctypes
import struct
from typing import Optional

import numpy as np
import torch

from .. import _native as N
from ..ops import interleave_gate_up
from ..ops.megakernel import BM, COMM_REDUCE_LOCAL, ProgramBuilder, RowEvents, _pack_comm, _pack_elt
from ..parallel import fused
from ..parallel.symm_heap import LocalHeap
from ..task_graph.nodes import TaskType

T_TOPK, T_MOE_RETURN, T_MOE_COUNTS, T_MOE_COMBINE, T_FILL = 110, 116, 117, 119, 301


def heap_bytes_needed(hidden: int, experts: int, top_k: int, tokens: int, world: int, capacity: int) -> int:
    el = experts // world
    return (el * world * capacity * (hidden * 2 + 16) + world * el * 4 + tokens * top_k * hidden * 2 + (8 << 20))


class MoEEPLayer:
    def __init__(self, hidden: int = 2048, experts: int = 128, top_k: int = 8, inter: int = 768, tokens: int = 4096, *,
                 rank: int = 0, world: int = 1, heap=None, device: Optional[torch.device] = None,
                 dtype: torch.dtype = torch.bfloat16, capacity_factor: float = 2.0, seed: int = 0, mode: str = "static",
                 trace: bool = False, weight_std: float = 0.02, router_std: float = 0.02, on_drop: str = "warn",
                 fused_return: Optional[bool] = None):
        import os
        # The weighted return of the expert outputs (the combine all-to-all) happens in the epilogue of the down
        # projection: every output row goes, scaled, straight into its source rank's combine buffer. Off: separate
        # MOE_RETURN tasks read the slab of outputs back and send the rows (they queue behind all expert tiles).
        self.fused_return = (os.environ.get("MACO_MOE_FUSED_RETURN", "1") != "0") if fused_return is None else bool(fused_return)
        if experts % world or tokens % BM or inter % 128 or hidden % 256:
            raise ValueError("experts % world, tokens % 128, inter % 128 and hidden % 256 must be 0")
        if top_k > 8 or experts > 256 or hidden * 2 * 4 > 20480:
            raise ValueError("supported: top_k <= 8, experts <= 256, hidden <= 2560")
        dev = self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.hidden, self.experts, self.top_k, self.inter, self.tokens = hidden, experts, top_k, inter, tokens
        self.rank, self.world, self.dtype = rank, world, dtype
        self.el = experts // world
        mean = tokens * top_k / experts
        self.capacity = max(BM, int(-(-mean * capacity_factor // BM)) * BM)
        if heap is None:
            if world > 1:
                raise ValueError("world > 1 needs the symmetric heap")
            heap = LocalHeap(heap_bytes_needed(hidden, experts, top_k, tokens, world, self.capacity), dev)
        self.heap = heap
        EL, W, C, H, I, T, K = self.el, world, self.capacity, hidden, inter, tokens, top_k
        g_shared = torch.Generator(device="cpu").manual_seed(seed * 131 + 7)
        self.w_router = (torch.randn(experts, H, generator=g_shared) * router_std).to(dtype).to(dev)
        # every expert's weights come from its own seed, so any rank can rebuild them for a check
        self._seed, self._wstd = seed, weight_std
        w1, w2 = [], []
        self.w_gate, self.w_up, self.w_down = [], [], []
        for el in range(EL):
            wg, wu, wd = self.expert_weights(rank * EL + el)
            self.w_gate.append(wg); self.w_up.append(wu); self.w_down.append(wd)
            w1.append(interleave_gate_up(wg, wu))
            w2.append(wd)
        self.w1 = torch.stack(w1)                                   # [EL, 2I, H], gate/up interleaved per 256 rows
        self.w2 = torch.stack(w2)                                   # [EL, H, I]
        self.x = torch.empty(T, H, device=dev, dtype=dtype)
        self.logits = torch.empty(T, experts, device=dev, dtype=dtype)
        self.counts = torch.zeros(experts + 1, device=dev, dtype=torch.int32)
        self.recv = heap.alloc((EL, W, C, H), dtype)
        self.meta = heap.alloc((EL, W, C, 4), torch.int32)
        self.cnt = heap.alloc((W, EL), torch.int32)
        self.comb = heap.alloc((T, K, H), dtype)
        self.act = torch.zeros(EL, W, C, I, device=dev, dtype=dtype)
        self.y = torch.zeros(EL, W, C, H, device=dev, dtype=dtype)
        self.out = torch.empty(T, H, device=dev, dtype=dtype)
        params = struct.pack("<QQQQQQQQQiiiiiiii", self.logits.data_ptr(), self.x.data_ptr(), self.counts.data_ptr(),
                             self.comb.data_ptr(), heap.offset_of(self.recv), heap.offset_of(self.meta),
                             heap.offset_of(self.cnt), heap.offset_of(self.comb), self.y.data_ptr(), H, experts, K, EL, C, T,
                             N.DTYPE_CODE[dtype], 0)
        self.d_params = torch.from_numpy(np.frombuffer(params, dtype=np.uint8).copy()).to(dev)
        # Dropped-pair count of the last step, delivered without a blocking read: every forward() copies the counter
        # into pinned host memory behind the launch, and the NEXT forward() (or dropped()) looks at it. A step that
        # dropped pairs therefore never goes unnoticed, and nothing waits for the GPU on the way.
        on_gpu = dev.type == "cuda"
        self._drop_host = torch.zeros(1, dtype=torch.int32).pin_memory() if on_gpu else torch.zeros(1, dtype=torch.int32)
        self._drop_event = torch.cuda.Event() if on_gpu else None
        self._drop_pending = False
        self.total_dropped = 0
        self.on_drop = on_drop
        self._build(mode, trace)

    def expert_weights(self, e: int):
        g = torch.Generator(device="cpu").manual_seed(self._seed * 100003 + 17 * e + 1)
        mk = lambda *s: (torch.randn(*s, generator=g) * self._wstd).to(self.dtype).to(self.device)
        return mk(self.inter, self.hidden), mk(self.inter, self.hidden), mk(self.hidden, self.inter)

    # ------------------------------------------------------------------ program
    def _build(self, mode: str, trace: bool) -> None:
        EL, W, C, H, I, T, K = self.el, self.world, self.capacity, self.hidden, self.inter, self.tokens, self.top_k
        dt = N.DTYPE_CODE[self.dtype]
        b = ProgramBuilder(self.device, mode=mode, heap=self.heap, trace=trace)
        pp = self.d_params.data_ptr()
        fence = fused.epoch_fence_event(b)
        # 0. clear this rank's slot counters (first task of the launch; everything that follows is ordered behind it)
        e_fill = b.new_event()
        b.add_task(T_FILL, _pack_elt(0, 0, 0, self.counts.data_ptr(), 0, 1, self.experts + 1, 2, 0, 0, i0=0), waits=[fence],
                   signals=[e_fill])
        # 1. router
        e_log = b.gemm(self.x, self.w_router, self.logits, bn=128, extra_waits=[(e_fill, 1, False, False)])
        # 2. top-k + dispatch: about one task per worker, a multiple of 4 tokens (one warp per token)
        e_disp_local = b.new_event()
        n_disp = 0
        tok_per = max(4, -(-(-(-T // b.num_workers)) // 4) * 4)
        for t0 in range(0, T, tok_per):
            nt = min(tok_per, T - t0)
            ev, cnt = e_log.for_rows(t0, t0 + nt)
            b.add_task(T_TOPK, _pack_elt(0, 0, pp, 0, t0, nt, H, dt, 0, 0), waits=[(ev, cnt, False, False)],
                       signals=[e_disp_local])
            n_disp += 1
        # 3. counts to the expert owners; every rank learns that every rank has dispatched
        e_disp = b.new_event()
        b.add_task(T_MOE_COUNTS, _pack_elt(0, 0, pp, 0, 0, 0, 0, dt, 0, 0), waits=[(e_disp_local, n_disp, False, False)],
                   signal_peer=-2, signal_peer_event=e_disp)
        arrived = (e_disp, W, True, False)
        # 4. expert GEMMs over the slabs, tiles guarded by the received counts; 5. weighted return
        e_ret = b.new_event()
        cnt_base = self.cnt.data_ptr()
        # Phase order matters with static queues: a worker that is handed a down-projection tile right
        # behind the gate/up tiles of the same slab would idle until those finish. All gate/up tiles come
        # first, then all down tiles, then the returns, so a dependent task is always far behind its producers.
        pairs = [(el, s) for el in range(EL) for s in range(W)]
        guards, acts, ys = {}, {}, {}
        for el, s in pairs:
            cptr = cnt_base + (s * EL + el) * 4
            guards[el, s] = (lambda mb, nb, cptr=cptr: dict(count_ptr=cptr, count_base=mb * BM))
            acts[el, s] = b.gemm(self.recv[el, s], self.w1[el], self.act[el, s], epilogue="swiglu", bn=256,
                                 extra_waits=[arrived], per_tile=guards[el, s])
        def emit_return(el: int, s: int) -> None:
            for rb in range(C // BM):
                ev, cnt = ys[el, s].for_rows(rb * BM, (rb + 1) * BM)
                b.add_task(T_MOE_RETURN, _pack_elt(0, 0, pp, 0, rb * BM, BM, H, dt, 0, 0, i0=el, i1=s),
                           waits=[(ev, cnt, False, False)], signal_peer=s, signal_peer_event=e_ret)

        # Returns are queued behind every expert tile. Interleaving them `lag` slabs behind their
        # down-projection tiles was tried, to send rows back under the remaining GEMM work: with static queues
        # a return that waits even briefly holds up the epilogues of its worker, and the layer got 28 % slower.
        # (Also tried without gain: pulling the next tile's expert weights into L2 with TMA prefetches.)
        if self.fused_return:
            comb_off = self.heap.offset_of(self.comb)
            meta_base = self.meta.data_ptr()
            n_tiles_down = H // 256
            for el, s in pairs:
                cptr = cnt_base + (s * EL + el) * 4
                epi = b.add_epilogue(0, H, self.dtype, C, H, mode="scatter_rows", aux_ptr=meta_base + ((el * W + s) * C) * 16,
                                     bias_type=K)

                def scatter(mb, nb, cptr=cptr, epi=epi, s=s):
                    return dict(count_ptr=cptr, count_base=mb * BM, epi=epi, peer=s, out_off=comb_off, signal_peer=s,
                                signal_peer_event=e_ret)

                ys[el, s] = b.gemm(self.act[el, s], self.w2[el], self.y[el, s], bn=256, a_ready=acts[el, s], per_tile=scatter)
            n_ret = W * EL * (C // BM) * n_tiles_down
        else:
            for el, s in pairs:
                ys[el, s] = b.gemm(self.act[el, s], self.w2[el], self.y[el, s], bn=256, a_ready=acts[el, s],
                                   per_tile=guards[el, s])
            for el, s in pairs:
                emit_return(el, s)
            n_ret = W * EL * (C // BM)
        # 6. combine: sum the k rows of every token (token blocks streamed through the idle operand ring)
        e_out = b.new_event()
        n_out = 0
        per = max(8, -(-T // b.num_workers))
        for t0 in range(0, T, per):
            b.add_task(T_MOE_COMBINE, _pack_elt(0, 0, pp, self.out.data_ptr(), t0, min(per, T - t0), H, dt, 0, 0),
                       waits=[(e_ret, n_ret, True, False)], signals=[e_out])
            n_out += 1
        fused.epoch_fence_signal(b, [(e_out, n_out, False, False)])
        # (a CPU device plans only: the task list stays in ``self.builder`` for host-side schedule checks)
        self.builder = b
        self.program = b.build() if self.device.type == "cuda" else None

    def forward(self, x: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """One step. ``on_drop`` ("warn", "raise", "ignore") says what happens when an EARLIER step turns out to have
        dropped routed pairs (a slab's capacity was exceeded, ``capacity_factor`` too small for the routing skew)."""
        self._poll_drops(wait=False)
        if x is not None:
            self.x.copy_(x, non_blocking=True)
        self.program.run(stream=stream)
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.stream(st):
            self._drop_host.copy_(self.counts[self.experts:self.experts + 1], non_blocking=True)
            self._drop_event.record(st)
        self._drop_pending = True
        return self.out

    __call__ = forward

    def _poll_drops(self, wait: bool) -> int:
        if not self._drop_pending:
            return int(self._drop_host[0])
        if wait:
            self._drop_event.synchronize()
        elif not self._drop_event.query():
            return -1
        self._drop_pending = False
        n = int(self._drop_host[0])
        if n > 0:
            self.total_dropped += n
            msg = (f"MoE layer dropped {n} routed (token, expert) pairs in its last step: a receive slab holds "
                   f"{self.capacity} rows per (source rank, expert); raise capacity_factor")
            if self.on_drop == "raise":
                raise RuntimeError(msg)
            if self.on_drop == "warn":
                import warnings
                warnings.warn(msg, RuntimeWarning, stacklevel=3)
        return n

    def dropped(self) -> int:
        """(token, expert) pairs of the last step that exceeded a slab's capacity. Waits only for that step's
        copy of the counter (an event), not for the device."""
        return self._poll_drops(wait=True)

    # ------------------------------------------------------------------ oracle
    def reference(self, x: torch.Tensor) -> torch.Tensor:
        """fp32 PyTorch result for this rank's tokens (rebuilds every expert's weights from its seed)."""
        F = torch.nn.functional
        bf = lambda t: t.to(self.dtype).float()
        xf = x.float()
        logits = bf(xf @ self.w_router.float().t())
        # same tie rule as the kernel: larger logit first, lower expert index on equal logits
        sval, sidx = torch.sort(logits, dim=-1, descending=True, stable=True)
        val, idx = sval[:, : self.top_k], sidx[:, : self.top_k]
        w = torch.softmax(val, dim=-1)
        out = torch.zeros_like(xf)
        for e in torch.unique(idx).tolist():
            wg, wu, wd = self.expert_weights(e)
            tok, k = (idx == e).nonzero(as_tuple=True)
            h = bf(F.silu(xf[tok] @ wg.float().t()) * (xf[tok] @ wu.float().t()))
            y = bf(h @ wd.float().t())
            out.index_add_(0, tok, bf(y * w[tok, k].unsqueeze(1)))
        return out
