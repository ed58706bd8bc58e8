"""Split-KV decode attention for grouped-query attention (head_dim 128, up to 8 query heads per KV
head). The kernel streams each K and V row once; see csrc/attention_decode.cuh. The reference has
no attention kernel (its example materialises softmax(QK^T)V, examples/test_overlap_attention.py:111-113).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native as N

_declared = False


def _lib():
    global _declared
    lib = N.lib()
    if not _declared:
        P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib.maco_attention_decode.restype = I
        lib.maco_attention_decode.argtypes = [P, P, P, P, P, I, I, I, I, I, I, I, LL, LL, F, P]
        lib.maco_attention_decode_scratch_bytes.restype = ctypes.c_ulonglong
        lib.maco_attention_decode_scratch_bytes.argtypes = [I, I, I, I]
        _declared = True
    return lib


def default_splits(batch: int, kv_heads: int, seq: int) -> int:
    """Enough (batch, head, split) tasks to cover the SMs about twice, at least 256 keys per split."""
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    want = max(1, (2 * sms + batch * kv_heads - 1) // (batch * kv_heads))
    return max(1, min(want, max(1, seq // 256), 32))


_tc_programs: dict = {}


def attention_decode_tensor_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, *,
                                 scale: Optional[float] = None, kv_len: Optional[int] = None) -> torch.Tensor:
    """Decode attention through the persistent kernel's tensor-core task (csrc/attention_decode.cuh): K/V
    streamed by TMA, both products on tcgen05, the key range cut into one equal share per SM. Contiguous
    16-bit ``q`` [B, Hq, 128], ``k``/``v`` [B, Hkv, S, 128], ``out`` [B, Hq, 128]. The program is built once per
    set of buffers (tensor maps and task table hold their addresses) and re-launched afterwards."""
    from .megakernel import ProgramBuilder
    key = (q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), tuple(q.shape), tuple(k.shape), q.dtype, scale, kv_len)
    prog = _tc_programs.get(key)
    if prog is None:
        if len(_tc_programs) >= 16:
            _tc_programs.pop(next(iter(_tc_programs)))
        b = ProgramBuilder(q.device)
        b.attention_decode(q, k, v, out, kv_len=kv_len, scale=scale, balance=True)
        prog = _tc_programs[key] = b.build()
    prog.run()
    return out


def attention_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
                     splits: Optional[int] = None, out: Optional[torch.Tensor] = None,
                     scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``q`` [B, Hq, 128], ``k``/``v`` [B, Hkv, S, 128] (last two dims contiguous) -> [B, Hq, 128].
    With a caller-provided ``out``, contiguous 16-bit tensors and no explicit ``splits`` / ``scratch`` the call
    goes to ``attention_decode_tensor_core`` (about four times the K/V rate of the CUDA-core kernel below)."""
    B, Hq, D = q.shape
    _, Hkv, S, _ = k.shape
    if (out is not None and splits is None and scratch is None and D == 128 and q.dtype in (torch.bfloat16, torch.float16)
            and Hq % Hkv == 0 and Hq // Hkv <= 8 and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
            and out.is_contiguous() and k.shape == v.shape):
        return attention_decode_tensor_core(q, k, v, out, scale=scale)
    if k.shape != v.shape or k.stride() != v.stride() or k.stride(3) != 1 or k.stride(2) != D:
        raise ValueError("k and v must share a [B, Hkv, S, 128] layout with contiguous rows")
    q = q.contiguous()
    splits = splits or default_splits(B, Hkv, S)
    lib = _lib()
    need = lib.maco_attention_decode_scratch_bytes(B, Hq, Hkv, splits)
    if scratch is None:
        scratch = torch.empty(need // 4, dtype=torch.float32, device=q.device)
    elif scratch.numel() * scratch.element_size() < need:
        raise ValueError(f"scratch too small: need {need} bytes")
    if out is None:
        out = torch.empty_like(q)
    rc = lib.maco_attention_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), scratch.data_ptr(), B, Hq,
                                   Hkv, S, D, splits, N.DTYPE_CODE[q.dtype], k.stride(0), k.stride(1),
                                   float(scale if scale is not None else D ** -0.5), N.current_stream_ptr())
    N.check(rc, "maco_attention_decode")
    return out
