"""The allocation-free decode-attention entry point, called through its exported C symbol.

For callers that cannot allocate device memory (a fixed memory plan, a serving loop that must stay
out of the allocator, a plug-in without an allocator), ``maco_attention_decode_static`` keeps the
split-KV scratch in a 4 MiB array inside the library. This test checks it against the allocating
entry point on two calls in a row (the second one reuses the array with the first call's contents
still in it) and checks that an oversized request is refused on the host without launching.
The file name sorts last so that it runs after every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from maco_b200 import _native
    lib = _native.lib()
    P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.maco_attention_decode_static.restype = I
    lib.maco_attention_decode_static.argtypes = [P, P, P, P, I, I, I, I, I, I, I, LL, LL, F, P]
    lib.maco_attention_decode.restype = I
    lib.maco_attention_decode.argtypes = [P, P, P, P, P, I, I, I, I, I, I, I, LL, LL, F, P]
    lib.maco_attention_decode_scratch_bytes.restype = ctypes.c_ulonglong
    lib.maco_attention_decode_scratch_bytes.argtypes = [I, I, I, I]
    lib.maco_last_error.restype = ctypes.c_char_p
    return lib


def _case(B, Hq, Hkv, S, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16, generator=g)
    return mk(B, Hq, 128), mk(B, Hkv, S, 128), mk(B, Hkv, S, 128)


def test_static_scratch_entry_matches_allocating_entry_twice():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for seed, (B, Hq, Hkv, S, splits) in enumerate([(8, 8, 1, 2048, 4), (5, 16, 2, 777, 3)]):
        q, k, v = _case(B, Hq, Hkv, S, seed)
        scale = 128 ** -0.5
        need = lib.maco_attention_decode_scratch_bytes(B, Hq, Hkv, splits)
        scratch = torch.empty(need // 4, dtype=torch.float32, device="cuda")
        ref = torch.empty_like(q)
        rc = lib.maco_attention_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), ref.data_ptr(), scratch.data_ptr(), B, Hq,
                                       Hkv, S, 128, splits, 0, k.stride(0), k.stride(1), scale, stream)
        assert rc == 0, lib.maco_last_error()
        out = torch.zeros_like(q)
        rc = lib.maco_attention_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Hq, Hkv, S, 128,
                                              splits, 0, k.stride(0), k.stride(1), scale, stream)
        assert rc == 0, lib.maco_last_error()
        torch.cuda.synchronize()
        assert torch.equal(out, ref)          # the same kernels on the same inputs: bit-identical
        # and both agree with plain PyTorch in fp32
        G = Hq // Hkv
        s = torch.einsum("bhgd,bhsd->bhgs", q.float().view(B, Hkv, G, 128), k.float()) * scale
        pt = torch.einsum("bhgs,bhsd->bhgd", torch.softmax(s, -1), v.float()).reshape(B, Hq, 128)
        torch.testing.assert_close(out.float(), pt, atol=1e-1, rtol=5e-2)


def test_static_scratch_entry_refuses_oversized_requests():
    lib = _lib()
    B, Hq, Hkv, S, splits = 64, 8, 1, 4096, 32          # 64 * 32 * 4160 B = 8.1 MiB > 4 MiB
    assert lib.maco_attention_decode_scratch_bytes(B, Hq, Hkv, splits) > (4 << 20)
    q = torch.zeros(1, device="cuda", dtype=torch.bfloat16)
    rc = lib.maco_attention_decode_static(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), B, Hq, Hkv, S, 128, splits,
                                          0, 0, 0, 1.0, None)
    assert rc != 0
    msg = lib.maco_last_error().decode()
    assert "scratch" in msg and "fewer splits" in msg
    torch.cuda.synchronize()


def test_static_scratch_entry_refuses_misaligned_operands_on_the_host():
    """The kernels read K / V with 16-byte vector loads: a misaligned pointer or stride is refused before any launch."""
    lib = _lib()
    B, Hq, Hkv, S, splits = 2, 8, 1, 256, 2
    q, k, v = _case(B, Hq, Hkv, S, 7)
    out = torch.empty_like(q)
    args = lambda kp, bs, hs: (q.data_ptr(), kp, v.data_ptr(), out.data_ptr(), B, Hq, Hkv, S, 128, splits, 0, bs, hs, 0.1, None)
    assert lib.maco_attention_decode_static(*args(k.data_ptr() + 2, k.stride(0), k.stride(1))) != 0
    assert "aligned" in lib.maco_last_error().decode()
    assert lib.maco_attention_decode_static(*args(k.data_ptr(), k.stride(0) + 4, k.stride(1))) != 0
    assert "strides" in lib.maco_last_error().decode()
    assert lib.maco_attention_decode_static(*args(k.data_ptr(), k.stride(0), k.stride(1))) == 0
    torch.cuda.synchronize()
