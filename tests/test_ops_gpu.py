"""CUDA operators against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.conftest import assert_close


def _ops():
    from maco_b200 import ops
    return ops


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 128, 64), (200, 328, 136), (1024, 512, 2048), (64, 1280, 5120)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_tcgen05_all_majors(dtype, shape, bn):
    ops = _ops()
    M, N, K = shape
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    b = torch.randn(N, K, device="cuda", dtype=dtype) * 0.1
    ref = a.float() @ b.float().t()
    scale = ref.abs().max().item()
    for ta, tb in [(False, False), (False, True), (True, False), (True, True)]:
        aa = a.t().contiguous() if ta else a
        bb = b.t().contiguous() if tb else b
        out = ops.gemm(aa, bb, trans_a=ta, trans_b=tb, bn=bn)
        assert (out.float() - ref).abs().max().item() <= 1e-2 * scale, (ta, tb)
    from maco_b200 import _native
    assert _native.status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(256, 256, 64), (200, 328, 136), (1024, 512, 2048), (384, 1280, 512), (2304, 768, 320)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_two_cta_tiles_all_majors(dtype, shape, bn):
    """Two-CTA tiles (tcgen05.mma.cta_group::2): every operand major, ragged edges, an odd number of row blocks
    (the pair's second CTA then works on rows past the end and stores nothing)."""
    ops = _ops()
    M, N, K = shape
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    b = torch.randn(N, K, device="cuda", dtype=dtype) * 0.1
    ref = a.float() @ b.float().t()
    scale = ref.abs().max().item()
    for ta, tb in [(False, False), (False, True), (True, False), (True, True)]:
        aa = a.t().contiguous() if ta else a
        bb = b.t().contiguous() if tb else b
        out = ops.gemm(aa, bb, trans_a=ta, trans_b=tb, bn=bn, cta_pair=True)
        assert (out.float() - ref).abs().max().item() <= 1e-2 * scale, (ta, tb)
    from maco_b200 import _native
    assert _native.status() == 0


def test_gemm_two_cta_tiles_swiglu_and_large():
    ops = _ops()
    dt = torch.bfloat16
    F = torch.nn.functional
    a = torch.randn(2048, 1024, device="cuda", dtype=dt)
    wg = torch.randn(1536, 1024, device="cuda", dtype=dt) * 0.05
    wu = torch.randn(1536, 1024, device="cuda", dtype=dt) * 0.05
    fused = ops.interleave_gate_up(wg, wu)
    ref = F.silu(a.float() @ wg.float().t()) * (a.float() @ wu.float().t())
    assert_close(ops.gemm(a, fused, epilogue="swiglu", cta_pair=True), ref, dt)
    # more tiles than CTA pairs: every pair walks several tiles (accumulator double buffer, ring wrap-around)
    a = torch.randn(4096, 512, device="cuda", dtype=dt)
    b = torch.randn(4096, 512, device="cuda", dtype=dt) * 0.05
    one = ops.gemm(a, b, cta_pair=False)
    two = ops.gemm(a, b, cta_pair=True)
    assert_close(two, a.float() @ b.float().t(), dt)
    assert torch.equal(one, two)          # same products, same accumulation order per output element
    from maco_b200 import _native
    assert _native.status() == 0


def test_gemm_epilogues():
    ops = _ops()
    M, N, K = 512, 1024, 512
    dt = torch.bfloat16
    a = torch.randn(M, K, device="cuda", dtype=dt)
    b = torch.randn(N, K, device="cuda", dtype=dt) * 0.05
    bias = torch.randn(N, device="cuda", dtype=dt)
    aux = torch.randn(M, N, device="cuda", dtype=dt)
    acc = a.float() @ b.float().t()
    F = torch.nn.functional
    assert_close(ops.gemm(a, b, bias=bias), acc + bias.float(), dt)
    assert_close(ops.gemm(a, b, bias=bias, epilogue="gelu"), F.gelu(acc + bias.float(), approximate="tanh"), dt)
    assert_close(ops.gemm(a, b, epilogue="silu"), F.silu(acc), dt)
    assert_close(ops.gemm(a, b, aux=aux, epilogue="residual"), acc + aux.float(), dt)
    o32 = ops.gemm(a, b, epilogue="f32", alpha=0.5)
    torch.testing.assert_close(o32, 0.5 * acc, atol=2e-3, rtol=2e-3)
    ops.gemm(a, b, epilogue="f32_acc", alpha=0.5, out=o32)
    torch.testing.assert_close(o32, acc, atol=4e-3, rtol=4e-3)
    x = aux.float().requires_grad_(True)
    F.gelu(x, approximate="tanh").sum().backward()
    assert_close(ops.gemm(a, b, aux=aux, epilogue="gelu_bwd"), acc * x.grad, dt)
    wg, wu = b[: N // 2], b[N // 2:]
    fused = ops.interleave_gate_up(wg.contiguous(), wu.contiguous())
    ref = F.silu(a.float() @ wg.float().t()) * (a.float() @ wu.float().t())
    assert_close(ops.gemm(a, fused, epilogue="swiglu"), ref, dt)


def test_gemm_fp32_on_tensor_cores_as_tf32_is_opt_in():
    """fp32 operands: CUDA-core fp32 by default (1e-4), tcgen05 kind::tf32 with config.allow_tf32 (TF32 accuracy)."""
    import maco_b200 as maco
    ops = _ops()
    a = torch.randn(300, 520, device="cuda")
    w = torch.randn(264, 520, device="cuda") * 0.1
    bias = torch.randn(264, device="cuda")
    ref = torch.nn.functional.linear(a.double(), w.double(), bias.double()).float()
    torch.testing.assert_close(ops.linear(a, w, bias), ref, atol=1e-4, rtol=1e-4)
    maco.config.set(allow_tf32=True)
    try:
        out = ops.linear(a, w, bias)
        big = ops.gemm(torch.randn(1024, 2048, device="cuda"), torch.randn(1536, 2048, device="cuda"))
    finally:
        maco.config.set(allow_tf32=False)
    err = (out - ref).abs().max().item()
    assert 1e-6 < err < 3e-2, err          # TF32 rounding is visible, and bounded
    from maco_b200 import _native
    assert _native.status() == 0 and torch.isfinite(big).all()


def test_gemm_fp32_simt_and_odd_shapes():
    ops = _ops()
    a = torch.randn(33, 70, device="cuda")
    b = torch.randn(70, 45, device="cuda")
    torch.testing.assert_close(ops.matmul(a, b), a @ b, atol=1e-4, rtol=1e-4)
    w = torch.randn(45, 70, device="cuda")
    bias = torch.randn(45, device="cuda")
    torch.testing.assert_close(ops.linear(a, w, bias), torch.nn.functional.linear(a, w, bias), atol=1e-4, rtol=1e-4)
    # 16-bit inputs whose rows are not 16-byte aligned take the CUDA-core kernel too
    ah, bh = a.half(), w.half()
    assert_close(ops.linear(ah, bh), ah.float() @ bh.float().t(), torch.float16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(37, 256), (513, 1000), (4, 8192)])
def test_elementwise_and_rowwise(dtype, shape):
    ops = _ops()
    F = torch.nn.functional
    x = torch.randn(*shape, device="cuda", dtype=dtype)
    y = torch.randn(*shape, device="cuda", dtype=dtype)
    w = torch.randn(shape[1], device="cuda", dtype=dtype)
    b = torch.randn(shape[1], device="cuda", dtype=dtype)
    xf, yf = x.float(), y.float()
    assert_close(ops.gelu(x), F.gelu(xf, approximate="tanh"), dtype)
    assert_close(ops.silu(x), F.silu(xf), dtype)
    assert_close(ops.scale(x, 0.25), xf * 0.25, dtype)
    assert_close(ops.add(x, y), xf + yf, dtype)
    assert_close(ops.silu_gate(x, y), F.silu(xf) * yf, dtype)
    assert_close(ops.softmax(x), torch.softmax(xf, -1), dtype)
    assert_close(ops.rmsnorm(x, w, 1e-6), xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float(), dtype)
    assert_close(ops.layernorm(x, w, b, 1e-5), F.layer_norm(xf, (shape[1],), w.float(), b.float(), 1e-5), dtype)
    g = yf.clone().requires_grad_(True)
    F.gelu(g, approximate="tanh").sum().backward()
    assert_close(ops.gelu_bwd(x, y), xf * g.grad, dtype)


def test_rope_and_qknorm_rope():
    ops = _ops()
    from maco_b200.task_graph.runtime import rope_reference
    tokens, heads, hd = 64, 8, 128
    x = torch.randn(tokens, heads, hd, device="cuda", dtype=torch.bfloat16)
    ang = torch.randn(tokens, hd // 2, device="cuda")
    cos, sin = ang.cos(), ang.sin()
    assert_close(ops.rope(x, cos, sin), rope_reference(x.float(), cos, sin), torch.bfloat16)
    w = torch.randn(hd, device="cuda", dtype=torch.bfloat16)
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    cs = torch.cat([cos, sin], -1)
    assert_close(ops.qknorm_rope(x, w, cs, 1e-6), rope_reference(xn, cos, sin), torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg", [(4, 8, 1, 1000, 4), (2, 16, 2, 4097, None), (3, 4, 4, 130, 1)])
def test_attention_decode(dtype, cfg):
    ops = _ops()
    B, Hq, Hkv, S, splits = cfg
    q = torch.randn(B, Hq, 128, device="cuda", dtype=dtype)
    k = torch.randn(B, Hkv, S, 128, device="cuda", dtype=dtype)
    v = torch.randn(B, Hkv, S, 128, device="cuda", dtype=dtype)
    out = ops.attention_decode(q, k, v, splits=splits)
    G = Hq // Hkv
    qf = q.float().view(B, Hkv, G, 128)
    s = torch.einsum("bhgd,bhsd->bhgs", qf, k.float()) * 128 ** -0.5
    ref = torch.einsum("bhgs,bhsd->bhgd", torch.softmax(s, -1), v.float()).reshape(B, Hq, 128)
    assert_close(out, ref, dtype)
    # the same call with a caller-provided output and no split count goes through the tensor-core task of the
    # persistent kernel (fp16 and bf16; twice: the program is cached per set of buffers)
    out2 = torch.empty_like(q)
    for _ in range(2):
        out2.zero_()
        ops.attention_decode(q, k, v, out=out2)
        torch.cuda.synchronize()
        assert_close(out2, ref, dtype)
