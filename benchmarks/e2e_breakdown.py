#!/usr/bin/env python
"""Where an end-to-end step of the tensor-parallel layer spends its time beyond the kernel.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/e2e_breakdown.py

Times (CUDA events, max over ranks, microseconds per step) of the same layer step with more and more of the
end-to-end work around it: the kernel alone back to back; kernel + host synchronise; + device -> host read of the
result; + the device-to-device delivery of a staged input; a host -> device copy running on a side stream with NO
dependency on the step (pure interference); the full synchronous loop; the pipelined loop (``StepPipeline``).
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist


def main():
    rank, local, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    import maco_b200 as maco
    from maco_b200.models.tp_mlp import TPSwiGLUMLP
    from maco_b200.parallel import symm_heap
    from maco_b200.utils import InputPrefetcher, StepPipeline
    T, H, F = 8192, 4096, 14336
    heap = None
    if world > 1:
        maco.config.set(comm_buffer_size=str(int(T * H * 2 * (2 + 1.0 / world)) + (64 << 20)), backend="peer")
        maco.init(backend="nccl")
        heap = symm_heap.current_heap()
    layer = TPSwiGLUMLP(T, H, F, rank=rank, world=world, heap=heap, seed=0)
    rows = T // world
    x_host = torch.randn(rows, H).to(torch.bfloat16).pin_memory()
    dbuf = x_host.cuda()
    layer.x_shard.copy_(x_host)          # the same N(0,1) data as the benchmark in every variant
    res_host = torch.zeros(2, dtype=torch.bfloat16).pin_memory()
    side = torch.cuda.Stream()

    def tm(fn, steps=20, warm=3, finish=None):
        for _ in range(warm):
            fn()
        if finish:
            finish()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if finish:
            finish()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps * 1e3], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(float(t.item()), 1)

    sync = lambda: torch.cuda.current_stream().synchronize()
    out = {"n_gpus": world, "h2d_bytes_per_step": x_host.numel() * 2}
    out["h2d_copy_alone_us"] = tm(lambda: dbuf.copy_(x_host, non_blocking=True))
    out["kernel_back_to_back_us"] = tm(lambda: layer.forward(None))

    def fwd_sync():
        layer.forward(None); sync()
    out["kernel_then_host_sync_us"] = tm(fwd_sync)

    def fwd_read_sync():
        y = layer.forward(None)
        res_host.copy_(y[0, :2], non_blocking=True); sync()
    out["plus_result_read_us"] = tm(fwd_read_sync)

    def d2d_fwd_read_sync():
        layer.x_shard.copy_(dbuf, non_blocking=True)
        y = layer.forward(None)
        res_host.copy_(y[0, :2], non_blocking=True); sync()
    out["plus_input_delivery_us"] = tm(d2d_fwd_read_sync)

    def interference():
        layer.forward(None)
        with torch.cuda.stream(side):
            dbuf.copy_(x_host, non_blocking=True)
        sync()
    out["kernel_sync_with_unrelated_h2d_us"] = tm(interference)
    feed = InputPrefetcher(layer.x_shard)

    def synchronous_e2e():
        if not feed.pending:
            feed.submit(x_host)
        feed.deliver(layer.x_shard)
        y = layer.forward(None)
        feed.submit(x_host)
        res_host.copy_(y[0, :2], non_blocking=True); sync()
    out["synchronous_e2e_us"] = tm(synchronous_e2e)
    pipe = StepPipeline(layer.x_shard, layer.y_shard[0, :2])
    out["pipelined_e2e_us"] = tm(lambda: pipe.step(x_host, lambda: layer.forward(None), lambda: layer.y_shard[0, :2]),
                                 finish=pipe.drain)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        maco.cleanup()


if __name__ == "__main__":
    main()
