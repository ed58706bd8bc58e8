"""GEMM operators: the tcgen05 pipeline for 16-bit inputs, a CUDA-core kernel for the rest.

``linear`` / ``matmul`` are what ``TaskGraph.linear`` / ``TaskGraph.matmul`` lower to when a node
runs as its own launch; they replace the ``torch.mm`` calls of the reference's live runtime
(maco/task_graph/runtime.py:188-209) with this package's own kernels.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N

EPI_STORE, EPI_GELU, EPI_SWIGLU, EPI_F32_STORE, EPI_F32_ACC, EPI_GELU_BWD, EPI_SILU, EPI_RESIDUAL = range(8)

_MODES = {
    None: EPI_STORE, "none": EPI_STORE, "gelu": EPI_GELU, "swiglu": EPI_SWIGLU, "f32": EPI_F32_STORE,
    "f32_acc": EPI_F32_ACC, "gelu_bwd": EPI_GELU_BWD, "silu": EPI_SILU, "residual": EPI_RESIDUAL,
}


def _row_major_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError(f"expected a 2-D tensor, got {tuple(t.shape)}")
    if t.stride(1) != 1:
        t = t.contiguous()
    return t


def _tma_ok(t: torch.Tensor) -> bool:
    return t.data_ptr() % 16 == 0 and (t.stride(0) * t.element_size()) % 16 == 0 and t.stride(1) == 1


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    trans_a: bool = False,
    trans_b: bool = False,
    out: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    aux: Optional[torch.Tensor] = None,
    epilogue: Optional[str] = None,
    alpha: float = 1.0,
    out_dtype: Optional[torch.dtype] = None,
    bn: int = 0,
    max_ctas: int = 0,
    wait_budget_ms: float = 0.0,
    stream: Optional[torch.cuda.Stream] = None,
    cta_pair: Optional[bool] = None,
) -> torch.Tensor:
    """``out = epilogue(alpha * A' @ B'^T)`` with ``A' = a.T if trans_a else a`` (shape [M, K]) and
    ``B' = b.T if trans_b else b`` (shape [N, K]).

    ``trans_*`` describe how the operand is *stored*: ``trans_a`` means ``a`` is [K, M] row-major,
    ``trans_b`` means ``b`` is [K, N] row-major (the plain ``a @ b`` case). No copy is made for
    either layout: the MMA reads MN-major operands directly from shared memory.
    ``cta_pair``: True runs two-CTA tiles (``tcgen05.mma.cta_group::2``, 256 x bn per CTA pair), False one-CTA
    tiles (128 x bn), None lets the launcher choose (pairs once the tiles cover every SM pair).
    """
    if not a.is_cuda:
        raise ValueError("maco_b200.ops.gemm needs CUDA tensors")
    a = _row_major_2d(a)
    b = _row_major_2d(b)
    M, K = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    Nn, Kb = (b.shape[1], b.shape[0]) if trans_b else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    if a.dtype != b.dtype:
        raise ValueError(f"operand dtypes differ: {a.dtype} vs {b.dtype}")
    mode = _MODES[epilogue]
    n_out = Nn // 2 if mode == EPI_SWIGLU else Nn
    if out is None:
        od = out_dtype or (torch.float32 if mode in (EPI_F32_STORE, EPI_F32_ACC) else a.dtype)
        out = torch.empty((M, n_out), device=a.device, dtype=od)
    if out.dim() != 2 or out.shape[0] != M or out.shape[1] != n_out or out.stride(1) != 1:
        raise ValueError(f"out must be a row-major [{M}, {n_out}] tensor, got {tuple(out.shape)}")
    if M == 0 or Nn == 0:
        return out
    if K == 0:
        if mode != EPI_F32_ACC:
            out.zero_()
        return out
    lib = N.lib()
    st = N.current_stream_ptr(stream)
    bias_t = N.DTYPE_CODE[bias.dtype] if bias is not None else 0
    aux_t = N.DTYPE_CODE[aux.dtype] if aux is not None else 0
    ld_aux = aux.stride(0) if aux is not None else 0
    fast = (
        a.dtype in (torch.bfloat16, torch.float16)
        and _tma_ok(a) and _tma_ok(b)
        and out.data_ptr() % 16 == 0 and (out.stride(0) * out.element_size()) % 16 == 0
    )
    if fast:
        rc = lib.maco_gemm(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, Nn, K, a.stride(0), b.stride(0), out.stride(0),
            int(trans_a), int(trans_b), N.DTYPE_CODE[a.dtype], N.DTYPE_CODE[out.dtype], mode, N.ptr(bias), bias_t,
            N.ptr(aux), ld_aux, aux_t, float(alpha), bn, max_ctas, float(wait_budget_ms), st,
            0 if cta_pair is None else (2 if cta_pair else 1),
        )
        if rc == 0:
            return out
        if rc != -2:
            N.check(rc, "maco_gemm")
    from ..config import config
    if (config.allow_tf32 and a.dtype == torch.float32 and not trans_a and not trans_b and mode != EPI_SWIGLU
            and _tma_ok(a) and _tma_ok(b) and out.data_ptr() % 16 == 0 and (out.stride(0) * out.element_size()) % 16 == 0):
        # opt-in: fp32 operands through tcgen05.mma.kind::tf32 (inputs rounded to 10 mantissa bits, fp32 accumulation)
        rc = lib.maco_gemm_tf32(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, Nn, K, a.stride(0), b.stride(0), out.stride(0),
                                N.DTYPE_CODE[out.dtype], mode, N.ptr(bias), bias_t, N.ptr(aux), ld_aux, aux_t, float(alpha),
                                max_ctas, float(wait_budget_ms), st)
        if rc == 0:
            return out
        if rc != -2:
            N.check(rc, "maco_gemm_tf32")
    if mode == EPI_SWIGLU:
        raise ValueError("the swiglu epilogue needs 16-bit, 16-byte aligned operands")
    sam, sak = (1, a.stride(0)) if trans_a else (a.stride(0), 1)
    sbn, sbk = (1, b.stride(0)) if trans_b else (b.stride(0), 1)
    rc = lib.maco_gemm_simt(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, Nn, K, sam, sak, sbn, sbk, out.stride(0),
        N.DTYPE_CODE[a.dtype], N.DTYPE_CODE[out.dtype], mode, N.ptr(bias), bias_t, N.ptr(aux), ld_aux, aux_t,
        float(alpha), st,
    )
    N.check(rc, "maco_gemm_simt")
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, epilogue: Optional[str] = None, **kw) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` for ``x`` of shape [..., K] and ``weight`` [N, K]."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    n_out = weight.shape[0] // 2 if epilogue == "swiglu" else weight.shape[0]
    out2 = out.view(-1, n_out) if out is not None else None
    res = gemm(x2, weight, out=out2, bias=bias, epilogue=epilogue, **kw)
    return out if out is not None else res.view(*lead, n_out)


def matmul(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
    """``a @ b`` for 2-D ``a`` [M, K] and ``b`` [K, N]; ``b`` is read in place (no transpose copy)."""
    return gemm(a, b, trans_b=True, out=out, **kw)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Builds the fused SwiGLU weight: rows are laid out as [gate block | up block] per 2*block rows
    so that one 256-column GEMM tile holds both projections of the same 128 output features and
    the epilogue can apply ``silu(gate) * up`` before anything is written to memory."""
    f, k = w_gate.shape
    if w_up.shape != w_gate.shape or f % block != 0:
        raise ValueError("gate/up weights must have equal shapes with out_features a multiple of 128")
    g = w_gate.view(f // block, 1, block, k)
    u = w_up.view(f // block, 1, block, k)
    return torch.cat([g, u], dim=1).reshape(2 * f, k).contiguous()


def block_weight(w: torch.Tensor, bn: int = 256, bk: int = 64) -> torch.Tensor:
    """Re-lays a K-major weight ``w`` [N, K] tile by tile: ``out[nb, kb] = w[nb*bn:(nb+1)*bn, kb*bk:(kb+1)*bk]``,
    shape [N / bn, K / bk, bn, bk], contiguous. A few-row (decode) GEMM reads every weight byte exactly once; in
    the plain layout one TMA box of a tile is ``bn`` separate 128-byte pieces, each on its own DRAM page, and the
    stream stays near 4.5 TB/s, where contiguous 32 KB blocks stream at the rate of a plain copy
    (``ProgramBuilder.gemm_splitk(..., w_blocked=...)``). Done once when the model is built."""
    n, k = w.shape
    if n % bn or k % bk:
        raise ValueError(f"block_weight: shape {tuple(w.shape)} is not a multiple of ({bn}, {bk})")
    return w.view(n // bn, bn, k // bk, bk).permute(0, 2, 1, 3).contiguous()


def unblock_weight(wb: torch.Tensor) -> torch.Tensor:
    """Inverse of ``block_weight``: back to [N, K]."""
    nb, kb, bn, bk = wb.shape
    return wb.permute(0, 2, 1, 3).reshape(nb * bn, kb * bk).contiguous()
