#!/usr/bin/env python
"""One decode step of a Qwen3-style layer as ONE launch of the persistent kernel.

    python examples/decode_layer.py                       # one GPU
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/decode_layer.py   # tensor parallel

Shows the pieces a decode step is made of: split-K projections (`ProgramBuilder.gemm_splitk`),
QK-norm + RoPE, tensor-core split-KV attention (`ProgramBuilder.attention_decode`), one-shot
all-reduce fused into the o-proj / down-proj finishing tasks.
The reference's counterpart is a list of separate torch calls (benchmarks/benchmark_inference.py:60-133).
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import maco_b200 as maco
from maco_b200.models.qwen3_layer import Qwen3DecodeLayer


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    heap = None
    if world > 1:
        maco.config.set(comm_buffer_size="64MB", backend="peer")
        maco.init(backend="nccl")
        from maco_b200.parallel import symm_heap
        heap = symm_heap.current_heap()
    layer = Qwen3DecodeLayer(hidden=2048, q_heads=16, kv_heads=4, ffn=8192, batch=16, kv_len=2048,
                             rank=rank, world=world, heap=heap, trace=True)
    torch.manual_seed(0)
    x = torch.randn(16, 2048, device="cuda", dtype=torch.bfloat16)
    allreduce = None
    if world > 1:
        import torch.distributed as dist

        def allreduce(t):
            dist.all_reduce(t)
            return t
    ref = layer.reference(x, allreduce)          # uses the cache as it is before the step
    y = layer(x)
    torch.cuda.synchronize()
    if rank == 0:
        st = layer.program.stats()
        print(f"decode step: {st['span_us']:.0f} us in one launch, {st['tasks']} tasks; max |y - ref| = "
              f"{(y.float() - ref).abs().max().item():.3e}")
        for name, rec in st["by_type"].items():
            print(f"  {name:12s} x{rec['count']:5d}  busy {rec['busy_us']:9.0f} us")
    if world > 1:
        maco.cleanup()


if __name__ == "__main__":
    main()
