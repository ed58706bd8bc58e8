"""Element-wise and row-wise operators backed by this package's CUDA kernels (csrc/elementwise.cuh).

These are the stand-alone launches; the same device code runs as tasks inside the persistent
kernel. Reference counterparts: the device tasks of maco/csrc/maco_worker.cuh:66-177.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native as N

T_LAYERNORM, T_RMSNORM, T_GELU, T_SILU, T_SOFTMAX, T_SILU_GATE, T_ROPE = 103, 104, 105, 106, 107, 108, 109
T_SCALE, T_ADD, T_GELU_BWD, T_AXPBY, T_COPY = 112, 113, 114, 115, 300

_declared = False


def _fn():
    global _declared
    lib = N.lib()
    if not _declared:
        P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lib.maco_elementwise.restype = I
        lib.maco_elementwise.argtypes = [I, P, P, P, P, I, I, I, I, I, F, F, I, I, P]
        _declared = True
    return lib.maco_elementwise


def _rows2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 0:
        t = t.reshape(1, 1)
    t2 = t.reshape(-1, t.shape[-1]) if t.is_contiguous() else t.contiguous().reshape(-1, t.shape[-1])
    return t2


def _launch(kind: int, x: torch.Tensor, in1=None, in2=None, out: Optional[torch.Tensor] = None, f0=0.0, f1=0.0,
            i0=0, i1=0, rows=None, cols=None, ld=None) -> torch.Tensor:
    if not x.is_cuda:
        raise ValueError("maco_b200 element-wise operators need CUDA tensors")
    if x.dtype not in N.DTYPE_CODE:
        raise ValueError(f"unsupported dtype {x.dtype}")
    xc = x if x.is_contiguous() else x.contiguous()
    if out is None:
        out = torch.empty_like(xc)
    if not out.is_contiguous():
        raise ValueError("out must be contiguous")
    if xc.numel() == 0:
        return out
    c = cols if cols is not None else xc.shape[-1]
    r = rows if rows is not None else xc.numel() // c
    a1 = in1.contiguous() if in1 is not None else None
    a2 = in2.contiguous() if in2 is not None else None
    ld = ld if ld is not None else c
    rc = _fn()(kind, xc.data_ptr(), N.ptr(a1), N.ptr(a2), out.data_ptr(), r, c, N.DTYPE_CODE[x.dtype], ld, ld,
               float(f0), float(f1), int(i0), int(i1), N.current_stream_ptr())
    N.check(rc, "maco_elementwise")
    return out


def gelu(x, out=None): return _launch(T_GELU, x, out=out)
def silu(x, out=None): return _launch(T_SILU, x, out=out)
def softmax(x, out=None): return _launch(T_SOFTMAX, x, out=out)
def scale(x, factor: float, out=None): return _launch(T_SCALE, x, out=out, f0=factor)
def add(a, b, out=None): return _launch(T_ADD, a, in1=b, out=out)
def silu_gate(gate, up, out=None): return _launch(T_SILU_GATE, gate, in1=up, out=out)
def gelu_bwd(dy, pre, out=None): return _launch(T_GELU_BWD, dy, in1=pre, out=out)
def axpby(x, y, a: float, b: float, out=None): return _launch(T_AXPBY, x, in1=y, out=out, f0=a, f1=b)
def rmsnorm(x, weight, eps: float = 1e-6, out=None): return _launch(T_RMSNORM, x, in1=weight, out=out, f0=eps)
def layernorm(x, weight, bias, eps: float = 1e-5, out=None):
    return _launch(T_LAYERNORM, x, in1=weight, in2=bias, out=out, f0=eps)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out=None) -> torch.Tensor:
    """Half-rotation RoPE on [tokens, heads, head_dim]; cos/sin are [tokens, head_dim // 2]."""
    tokens, heads, hd = x.shape
    return _launch(T_ROPE, x, in1=cos.to(x.dtype), in2=sin.to(x.dtype), out=out, i0=heads, i1=0,
                   rows=tokens * heads, cols=hd, ld=heads * hd)


def qknorm_rope(x: torch.Tensor, weight: torch.Tensor, cos_sin: torch.Tensor, eps: float = 1e-6, out=None,
                token_offset: int = 0) -> torch.Tensor:
    """Per-head RMSNorm then RoPE on [tokens, heads, head_dim]; ``cos_sin`` is [tokens, head_dim]
    with cos in the first half of each row and sin in the second."""
    tokens, heads, hd = x.shape
    return _launch(T_ROPE, x, in1=weight, in2=cos_sin.to(x.dtype), out=out, f0=eps, f1=1.0, i0=heads,
                   i1=token_offset, rows=tokens * heads, cols=hd, ld=heads * hd)
