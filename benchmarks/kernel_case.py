#!/usr/bin/env python
"""Small, self-ending single-GPU cases of the hot kernels, for profiler captures and quick timing.

    python benchmarks/kernel_case.py gemm        # stand-alone tcgen05 GEMM, 8192 x 4096 x 4096 bf16, one-CTA tiles
    python benchmarks/kernel_case.py gemm_pair   # the same GEMM on two-CTA tiles (cta_group::2, clusters of two)
    python benchmarks/kernel_case.py mlp         # persistent kernel: fused SwiGLU MLP, 4096 tokens, 4096 -> 14336/4
    python benchmarks/kernel_case.py gemm_gate_up / gemm_down  # the layer's two GEMMs as stand-alone two-CTA kernels
    python benchmarks/kernel_case.py mlp_full    # the benchmark's layer on one GPU: 8192 tokens, 4096 -> 14336 (two-CTA tiles)
    python benchmarks/kernel_case.py mlp_full_1cta  # the same with one-CTA tiles
    python benchmarks/kernel_case.py attention   # split-KV decode attention, batch 32, 4096 keys
    python benchmarks/kernel_case.py attention_tc  # persistent kernel: tensor-core decode attention, 512 tasks, 537 MB of KV
    python benchmarks/kernel_case.py decode_gemm # persistent kernel: split-K 64 x 5120 x 25600 gate/up projection with SwiGLU
    python benchmarks/kernel_case.py moe         # persistent kernel: MoE layer on one GPU (32 experts, top-4, 2048 tokens)
    python benchmarks/kernel_case.py rmsnorm     # row-wise kernel, 16384 x 8192 bf16

Each case holds well under 1 GB on the device, uses inputs larger than the 126 MB L2 where DRAM
figures matter, warms up twice and then runs the kernel three times between CUDA events, printing
the mean time and the achieved rate.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from maco_b200 import _native, ops


def timed(fn, iters=3, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    dt = torch.bfloat16
    if case in ("gemm", "gemm_pair"):
        M, N, K = 8192, 4096, 4096
        a = torch.randn(M, K, device="cuda", dtype=dt)
        b = torch.randn(N, K, device="cuda", dtype=dt) * 0.02
        out = torch.empty(M, N, device="cuda", dtype=dt)
        us = timed(lambda: ops.gemm(a, b, out=out, bn=256, cta_pair=(case == "gemm_pair")))
        print(f"{case} {M}x{N}x{K}: {us:.1f} us, {2 * M * N * K / us / 1e6:.0f} TFLOP/s")
    elif case == "mlp":
        from maco_b200.models.tp_mlp import TPSwiGLUMLP
        layer = TPSwiGLUMLP(4096, 4096, 3584)
        layer.x_shard.normal_()
        us = timed(lambda: layer.forward(None))
        print(f"persistent fused MLP 4096 tok 4096->3584: {us:.1f} us, {layer.flops() / us / 1e6:.0f} TFLOP/s")
    elif case in ("gemm_gate_up", "gemm_down"):
        # the two GEMMs of the benchmark's layer as stand-alone two-CTA kernels (DRAM traffic per GEMM)
        M, N, K = (8192, 28672, 4096) if case == "gemm_gate_up" else (8192, 4096, 14336)
        a = torch.randn(M, K, device="cuda", dtype=dt)
        b = torch.randn(N, K, device="cuda", dtype=dt) * 0.02
        epi = "swiglu" if case == "gemm_gate_up" else None
        out = torch.empty(M, N // 2 if epi else N, device="cuda", dtype=dt)
        us = timed(lambda: ops.gemm(a, b, out=out, bn=256, epilogue=epi, cta_pair=True))
        print(f"{case} {M}x{N}x{K}: {us:.1f} us, {2 * M * N * K / us / 1e6:.0f} TFLOP/s")
    elif case in ("prog_gate_up", "prog_down"):
        # the same two GEMMs, each as a one-node program of the persistent kernel (two-CTA tiles)
        from maco_b200.ops.megakernel import ProgramBuilder
        M, N, K = (8192, 28672, 4096) if case == "prog_gate_up" else (8192, 4096, 14336)
        a = torch.randn(M, K, device="cuda", dtype=dt)
        b = torch.randn(N, K, device="cuda", dtype=dt) * 0.02
        epi = "swiglu" if case == "prog_gate_up" else None
        out = torch.empty(M, N // 2 if epi else N, device="cuda", dtype=dt)
        pb = ProgramBuilder(torch.device("cuda"), cta_pair=True)
        pb.gemm(a, b, out, epilogue=epi)
        prog = pb.build()
        us = timed(prog.run)
        print(f"{case} {M}x{N}x{K}: {us:.1f} us, {2 * M * N * K / us / 1e6:.0f} TFLOP/s")
    elif case in ("mlp_full", "mlp_full_1cta"):
        from maco_b200.models.tp_mlp import TPSwiGLUMLP
        layer = TPSwiGLUMLP(8192, 4096, 14336, cta_pair=(case == "mlp_full"))
        layer.x_shard.normal_()
        us = timed(lambda: layer.forward(None))
        print(f"persistent fused MLP 8192 tok 4096->14336 ({'two' if layer.program.cta_pair else 'one'}-CTA tiles): {us:.1f} us, "
              f"{layer.flops() / us / 1e6:.0f} TFLOP/s")
    elif case == "attention":
        B, Hq, Hkv, S = 32, 8, 1, 4096
        q = torch.randn(B, Hq, 128, device="cuda", dtype=dt)
        k = torch.randn(B, Hkv, S, 128, device="cuda", dtype=dt)
        v = torch.randn(B, Hkv, S, 128, device="cuda", dtype=dt)
        out = torch.empty_like(q)
        scratch = torch.empty(1 << 20, device="cuda", dtype=torch.float32)
        us = timed(lambda: ops.attention_decode(q, k, v, out=out, scratch=scratch))
        print(f"attention decode B{B} S{S}: {us:.1f} us, {2 * k.numel() * 2 / us / 1e3:.0f} GB/s of KV")
    elif case == "attention_tc":
        from maco_b200.ops.megakernel import ProgramBuilder
        B, Hq, Hkv, S, splits = 64, 32, 4, 4096, 2
        q = torch.randn(B, Hq, 128, device="cuda", dtype=dt)
        k = torch.randn(B, Hkv, S, 128, device="cuda", dtype=dt)
        v = torch.randn(B, Hkv, S, 128, device="cuda", dtype=dt)
        out = torch.empty_like(q)
        pb = ProgramBuilder(torch.device("cuda"), )
        pb.attention_decode(q, k, v, out, splits=splits)
        prog = pb.build()
        us = timed(prog.run)
        print(f"persistent tensor-core attention B{B} hq{Hq} hkv{Hkv} S{S} splits{splits}: {us:.1f} us, "
              f"{2 * k.numel() * 2 / us / 1e3:.0f} GB/s of KV")
        G = Hq // Hkv
        ref = torch.softmax(torch.einsum("bhgd,bhsd->bhgs", q[:4].float().view(4, Hkv, G, 128), k[:4].float()) * 128 ** -0.5, -1)
        ref = torch.einsum("bhgs,bhsd->bhgd", ref, v[:4].float()).reshape(4, Hq, 128)
        err = (out[:4].float() - ref).abs().max().item()
        print(f"max abs error against fp32 PyTorch (4 sequences): {err:.2e}")
        assert err < 2e-2
    elif case == "decode_gemm":
        from maco_b200.ops import interleave_gate_up
        from maco_b200.ops.megakernel import ProgramBuilder
        M, K, F = 64, 5120, 12800
        x = torch.randn(M, K, device="cuda", dtype=dt)
        wg = torch.randn(F, K, device="cuda", dtype=dt) * 0.02
        wu = torch.randn(F, K, device="cuda", dtype=dt) * 0.02
        w = interleave_gate_up(wg, wu, block=128)
        out = torch.empty(M, F, device="cuda", dtype=dt)
        pb = ProgramBuilder(torch.device("cuda"))
        pb.gemm_splitk(x, w, out, epilogue="swiglu")
        prog = pb.build()
        us = timed(prog.run)
        print(f"persistent split-K decode GEMM {M}x{K}x{2 * F} + SwiGLU: {us:.1f} us, {w.numel() * 2 / us / 1e3:.0f} GB/s of weights")
        ref = torch.nn.functional.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())
        err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
        print(f"max error relative to the largest output, against fp32 PyTorch: {err:.2e}")
        assert err < 2e-2
    elif case == "moe":
        from maco_b200.models.moe_layer import MoEEPLayer
        layer = MoEEPLayer(hidden=2048, experts=32, top_k=4, inter=768, tokens=2048, router_std=0.05)
        x = torch.randn(2048, 2048, device="cuda", dtype=dt)
        layer.x.copy_(x)
        us = timed(lambda: layer.forward(None))
        ref = layer.reference(x)
        err = ((layer.out.float() - ref).abs().max() / ref.abs().max()).item()
        print(f"persistent MoE layer 2048 tok, 32 experts top-4: {us:.1f} us, dropped {layer.dropped()}, max rel error {err:.2e}")
        assert err < 3e-2
    elif case == "rmsnorm":
        x = torch.randn(16384, 8192, device="cuda", dtype=dt)
        w = torch.randn(8192, device="cuda", dtype=dt)
        out = torch.empty_like(x)
        us = timed(lambda: ops.rmsnorm(x, w, 1e-6, out=out))
        print(f"rmsnorm 16384x8192: {us:.1f} us, {2 * x.numel() * 2 / us / 1e3:.0f} GB/s")
    else:
        raise SystemExit(f"unknown case {case}")
    assert _native.status() == 0


if __name__ == "__main__":
    main()
