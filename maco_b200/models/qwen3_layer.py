"""Qwen3-style decoder layer, decode step (one new token per sequence), tensor parallel.

    h1 = rmsnorm(x)                       q,k,v = h1 Wqkv^T           (heads split over ranks)
    q,k = rope(rmsnorm_per_head(q,k))     K,V cache[pos] = k,v      (in the finishing pass of the QKV projection)
    a   = attention(q, Kcache, Vcache)    o = a Wo^T   -> all-reduce, + x        = y1
    h2  = rmsnorm(y1)                     g = silu(h2 Wg^T) * (h2 Wu^T)
    d   = g Wd^T -> all-reduce, + y1      = out

One launch of the persistent kernel per rank runs the whole layer: every step above is a task
(GEMM tiles on tcgen05, QK-norm + RoPE, split-KV attention and its merge, RMSNorm), and both
all-reduces are fused into the producing GEMM: its epilogue stores each partial tile into every
rank's staging slot and bumps their counters, and each rank sums the slots (plus the residual) as
soon as they are complete, while the next task's weights are already being streamed.

The reference has no attention, RoPE or norm task and expresses a layer as separate torch calls
plus NCCL all-reduces (examples/tensor_parallel.py:95-112 skips attention altogether).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N
from ..ops import block_weight, interleave_gate_up
from ..ops.megakernel import BM, COMM_REDUCE_LOCAL, ProgramBuilder, RowEvents, _pack_comm, _pack_elt
from ..parallel import fused
from ..task_graph.nodes import TaskType

T_COPY = 300


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype: torch.dtype) -> torch.Tensor:
    """[tokens, head_dim] with cos in the first half of each row and sin in the second."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    ang = positions.float().unsqueeze(1) * inv.unsqueeze(0)
    return torch.cat([ang.cos(), ang.sin()], dim=1).to(dtype)


class Qwen3DecodeLayer:
    def __init__(self, hidden: int = 5120, q_heads: int = 64, kv_heads: int = 8, head_dim: int = 128, ffn: int = 25600,
                 batch: int = 64, kv_len: int = 4096, *, rank: int = 0, world: int = 1, heap=None,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16, theta: float = 1e6,
                 eps: float = 1e-6, seed: int = 0, mode: str = "static", trace: bool = False,
                 splits: Optional[int] = None, weight_std: float = 0.02, blocked_weights: bool = False,
                 fused_rope: Optional[bool] = None):
        import os
        self.fused_rope = (os.environ.get("MACO_QWEN3_FUSED_ROPE", "1") != "0") if fused_rope is None else bool(fused_rope)
        if head_dim != 128:
            raise ValueError("head_dim must be 128")
        if q_heads % world or kv_heads % world or ffn % (world * 64):
            raise ValueError("heads and ffn must divide by the world size (ffn by world*64)")
        if world > 1 and heap is None:
            raise ValueError("world > 1 needs the symmetric heap")
        self.hidden, self.D, self.batch, self.kv_len = hidden, head_dim, batch, kv_len
        self.rank, self.world, self.heap, self.dtype, self.eps, self.theta = rank, world, heap, dtype, eps, theta
        self.hq, self.hkv = q_heads // world, kv_heads // world
        self.G = self.hq // self.hkv
        if self.G > 8:
            raise ValueError("at most 8 query heads per KV head")
        self.f_local = ffn // world
        self.fused_rope = self.fused_rope and (self.hq + 2 * self.hkv) % 2 == 0 and batch <= BM   # whole 256-column tiles of heads
        dev = self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        B, H, D, hq, hkv = batch, hidden, head_dim, self.hq, self.hkv
        g = torch.Generator(device="cpu").manual_seed(seed * 1000 + rank)
        gs = torch.Generator(device="cpu").manual_seed(seed * 1000 + 999)      # shared across ranks
        mk = lambda gen, *s, std=weight_std: (torch.randn(*s, generator=gen) * std).to(dtype).to(dev)
        self.w_in = (1.0 + 0.1 * torch.randn(H, generator=gs)).to(dtype).to(dev)
        self.w_post = (1.0 + 0.1 * torch.randn(H, generator=gs)).to(dtype).to(dev)
        self.q_norm = (1.0 + 0.1 * torch.randn(D, generator=gs)).to(dtype).to(dev)
        self.k_norm = (1.0 + 0.1 * torch.randn(D, generator=gs)).to(dtype).to(dev)
        self.w_qkv = mk(g, (hq + 2 * hkv) * D, H)
        self.w_o = mk(g, H, hq * D)
        self.w_gate, self.w_up, self.w_down = mk(g, self.f_local, H), mk(g, self.f_local, H), mk(g, H, self.f_local)
        self.w_gate_up = interleave_gate_up(self.w_gate, self.w_up, block=128)   # 256-column tiles: gate 128 | up 128
        # ``blocked_weights``: tile-by-tile copies of the four projections, so that every TMA box is one contiguous
        # 32 KB block (the plain [N, K] tensors stay for the fp32 oracle). Off by default: measured no faster (the
        # K-major boxes already stream at the rate the consumers allow) and it doubles the weights' memory.
        self.blocked = blocked_weights and all(t.shape[0] % 256 == 0 and t.shape[1] % 64 == 0
                                               for t in (self.w_qkv, self.w_o, self.w_gate_up, self.w_down)) and batch <= BM
        blk = (lambda t: block_weight(t)) if self.blocked else (lambda t: None)
        self.wb_qkv, self.wb_o, self.wb_gate_up, self.wb_down = blk(self.w_qkv), blk(self.w_o), blk(self.w_gate_up), blk(self.w_down)
        self.S = kv_len + 1                                        # cache rows incl. the new token
        self.k_cache = mk(g, B, hkv, self.S, D, std=1.0)
        self.v_cache = mk(g, B, hkv, self.S, D, std=1.0)
        self.pos = kv_len
        self.cos_sin = rope_tables(torch.full((B,), float(self.pos), device=dev), D, theta, dtype)
        self.splits = splits or max(1, min(16, -(-2 * 148 // (B * hkv)), self.S // 256 or 1))
        e = lambda *s, dt=dtype: torch.empty(*s, device=dev, dtype=dt)
        self.x = e(B, H)
        self.h1, self.qkv, self.q_rot, self.attn = e(B, H), e(B, (hq + 2 * hkv) * D), e(B, hq, D), e(B, hq * D)
        self.y1, self.h2, self.act, self.out = e(B, H), e(B, H), e(B, self.f_local), e(B, H)
        if world > 1:
            self.slots1 = heap.alloc((world, B, H), dtype)
            self.slots2 = heap.alloc((world, B, H), dtype)
        self._build(mode, trace)

    # ------------------------------------------------------------------ program
    def _build(self, mode: str, trace: bool) -> None:
        B, H, D, hq, hkv, G, S = self.batch, self.hidden, self.D, self.hq, self.hkv, self.G, self.S
        dt = N.DTYPE_CODE[self.dtype]
        b = ProgramBuilder(self.device, mode=mode, heap=self.heap if self.world > 1 else None, trace=trace)
        fence = [fused.epoch_fence_event(b)] if self.world > 1 else []
        qw = (hq + 2 * hkv) * D
        e_h1 = b.elementwise(int(TaskType.RMSNORM), self.x, self.h1, in1=self.w_in, rows=B, cols=H, f0=self.eps,
                             extra_waits=fence)
        # the four projections are weight-streaming GEMMs with 64 rows: split-K tiles over every SM
        if self.fused_rope:
            # QK-norm, RoPE and the K / V cache update happen in the finishing pass of the projection itself: no QKV
            # buffer, no separate tasks, one dependency hop less before attention
            e_qkv = b.gemm_splitk(self.h1, self.w_qkv, None, epilogue="qk_rope", a_ready=e_h1, w_blocked=self.wb_qkv,
                                  rope=dict(q_out=self.q_rot, k_cache=self.k_cache, v_cache=self.v_cache, q_norm=self.q_norm,
                                            k_norm=self.k_norm, cos_sin=self.cos_sin, hq=hq, hkv=hkv, pos=self.pos, eps=self.eps))
            ready = [(e_qkv.all_event[0], e_qkv.all_event[1], False, False)]
        else:
            ready = self._rope_tasks(b, e_h1)
        self._rest_of_layer(b, ready, mode)

    def _rope_tasks(self, b, e_h1):
        B, H, D, hq, hkv, G, S = self.batch, self.hidden, self.D, self.hq, self.hkv, self.G, self.S
        qw = (hq + 2 * hkv) * D
        e_qkv = b.gemm_splitk(self.h1, self.w_qkv, self.qkv, a_ready=e_h1, w_blocked=self.wb_qkv)
        qkv_done = (e_qkv.all_event[0], e_qkv.all_event[1], False, False)
        # QK-norm + RoPE: q into its own buffer, k straight into the cache row of the new token, v copied
        # beside it. All of it bumps one event, so the attention tasks carry a single wait condition; task
        # sizes are chosen for few tasks per worker (each costs a few us of fixed latency).
        e_rope = b.new_event()
        n_rope = 0
        e_q = b.elementwise(int(TaskType.ROPE), self.qkv[:, : hq * D], self.q_rot, in1=self.q_norm, in2=self.cos_sin,
                            rows=B * hq, cols=D, f0=self.eps, f1=1.0, i0=hq, i1=0, ld_in=qw, ld_out=hq * D,
                            extra_waits=[qkv_done], rows_per_task=16 if B * hq >= 16 * b.num_workers // 2 else 4,
                            all_event=e_rope)
        n_rope += e_q.all_event[1]
        for j in range(hkv):
            e_k = b.elementwise(int(TaskType.ROPE), self.qkv[:, (hq + j) * D:(hq + j + 1) * D], self.k_cache[:, j, self.pos, :],
                                in1=self.k_norm, in2=self.cos_sin, rows=B, cols=D, f0=self.eps, f1=1.0, i0=1, i1=0,
                                ld_in=qw, ld_out=hkv * S * D, extra_waits=[qkv_done], rows_per_task=4, all_event=e_rope)
            e_v = b.elementwise(T_COPY, self.qkv[:, (hq + hkv + j) * D:(hq + hkv + j + 1) * D], self.v_cache[:, j, self.pos, :],
                                rows=B, cols=D, ld_in=qw, ld_out=hkv * S * D, extra_waits=[qkv_done], rows_per_task=B,
                                all_event=e_rope)
            n_rope += e_k.all_event[1] + e_v.all_event[1]
        return [(e_rope, n_rope, False, False)]

    def _rest_of_layer(self, b, ready, mode):
        B, H, D, hq, hkv, G, S = self.batch, self.hidden, self.D, self.hq, self.hkv, self.G, self.S
        # split-KV attention on the tensor cores: one task per (sequence, kv head, split), then the merges
        merged, n_merged = b.attention_decode(self.q_rot.view(B, hq, D), self.k_cache, self.v_cache, self.attn.view(B, hq, D),
                                              kv_len=S, splits=self.splits, waits=ready, balance=(mode == "static"))
        e_attn = RowEvents(rows=B, block=BM, row_events=[(merged, n_merged)], all_event=(merged, n_merged))
        slots1 = self.slots1 if self.world > 1 else None
        slots2 = self.slots2 if self.world > 1 else None
        e_y1 = fused.gemm_allreduce(b, self.attn, self.w_o, slots1, self.y1, residual=self.x, a_ready=e_attn,
                                    w_blocked=self.wb_o)
        e_h2 = b.elementwise(int(TaskType.RMSNORM), self.y1, self.h2, in1=self.w_post, rows=B, cols=H, f0=self.eps,
                             in_ready=[e_y1])
        e_act = b.gemm_splitk(self.h2, self.w_gate_up, self.act, epilogue="swiglu", a_ready=e_h2, w_blocked=self.wb_gate_up)
        e_out = fused.gemm_allreduce(b, self.act, self.w_down, slots2, self.out, residual=self.y1, a_ready=e_act,
                                     w_blocked=self.wb_down)
        if self.world > 1:
            fused.epoch_fence_signal(b, [(e_out.all_event[0], e_out.all_event[1], False, False)])
        # (a CPU device plans only: the task list stays in ``self.builder`` for host-side schedule checks)
        self.builder = b
        self.program = b.build() if self.device.type == "cuda" else None

    def forward(self, x: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """One decode step for ``x`` [batch, hidden] (copied into ``self.x``; None = already there)."""
        if x is not None:
            self.x.copy_(x, non_blocking=True)
        self.program.run(stream=stream)
        return self.out

    __call__ = forward

    def bytes_streamed(self) -> int:
        """Weights plus the KV cache rows one step has to read, per rank."""
        w = sum(t.numel() for t in (self.w_qkv, self.w_o, self.w_gate_up, self.w_down)) * 2
        return w + 2 * self.batch * self.hkv * self.S * self.D * 2

    # ------------------------------------------------------------------ oracle
    def reference(self, x: torch.Tensor, allreduce=None) -> torch.Tensor:
        """fp32 PyTorch result of the layer. ``allreduce(t)`` sums a tensor over ranks (None: one rank).
        Uses the cache contents BEFORE the step (the new token's k, v are computed here)."""
        F = torch.nn.functional
        B, H, D, hq, hkv, G = self.batch, self.hidden, self.D, self.hq, self.hkv, self.G
        ar = allreduce if allreduce is not None else (lambda t: t)
        rms = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + self.eps) * w.float()
        bf = lambda t: t.to(self.dtype).float()
        xf = x.float()
        h1 = bf(rms(xf, self.w_in))
        qkv = bf(h1 @ self.w_qkv.float().t())
        q = qkv[:, : hq * D].view(B, hq, D)
        k = qkv[:, hq * D:(hq + hkv) * D].view(B, hkv, D)
        v = qkv[:, (hq + hkv) * D:].view(B, hkv, D)
        cs = self.cos_sin.float()
        cos, sin = cs[:, : D // 2].unsqueeze(1), cs[:, D // 2:].unsqueeze(1)

        def norm_rope(t, w):
            t = rms(t, w)
            t1, t2 = t[..., : D // 2], t[..., D // 2:]
            return bf(torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1))

        q, k = norm_rope(q, self.q_norm), norm_rope(k, self.k_norm)
        kc, vc = self.k_cache.float().clone(), self.v_cache.float().clone()
        kc[:, :, self.pos], vc[:, :, self.pos] = k, v
        s = torch.einsum("bhgd,bhsd->bhgs", q.view(B, hkv, G, D), kc) * D ** -0.5
        a = bf(torch.einsum("bhgs,bhsd->bhgd", torch.softmax(s, -1), vc).reshape(B, hq * D))
        y1 = bf(ar(bf(a @ self.w_o.float().t())) + xf)
        h2 = bf(rms(y1, self.w_post))
        act = bf(F.silu(h2 @ self.w_gate.float().t()) * (h2 @ self.w_up.float().t()))
        return bf(ar(bf(act @ self.w_down.float().t())) + y1)
