#!/usr/bin/env python
"""Stand-alone collectives: this package's in-kernel forms against NCCL, and the overlap-efficiency figure.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/bench_collectives.py [--out collectives_N.jsonl]

* all-reduce sweep (fp32, 4 KB .. 64 MB): NCCL, peer pushes through staging slots, and (on a multicast-bound
  heap) multimem.ld_reduce / multimem.st through the NVSwitch;
* all-to-all sweep (equal splits): NCCL all_to_all_single against peer pushes;
* overlap efficiency = (t_comm + t_compute - t_overlapped) / min(t_comm, t_compute) for a 16 MB fp32 all-reduce
  next to a GEMM on a second stream, the figure the reference quotes as 92.2 % for NCCL on an L20
  (examples/benchmark_nccl_2gpu.py:148-213), here for NCCL + cuBLAS and for this package's all-reduce + GEMM.

Every number is device-timed (CUDA events, warm-up first) and the maximum over ranks. One JSON line per row.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist


def timed(fn, iters=20, warm=5, streams=()):
    for _ in range(warm):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    for s in streams:
        torch.cuda.current_stream().wait_stream(s)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--max-mb", type=int, default=64)
    args = ap.parse_args()
    rank, local, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    import maco_b200 as maco
    from maco_b200 import _native, ops
    from maco_b200.parallel import collectives, symm_heap
    maco.config.set(comm_buffer_size=f"{4 * args.max_mb + 256}MB", backend="peer")
    maco.init(backend="nccl")
    heap = symm_heap.current_heap()
    rows = []

    def emit(**kw):
        kw.update(world=world, heap=heap.mode + ("+multicast" if heap.multicast_base() else ""))
        rows.append(kw)
        if rank == 0:
            print(json.dumps(kw), flush=True)

    sizes = [4 << 10, 64 << 10, 640 << 10, 1 << 20, 16 << 20, args.max_mb << 20]
    for nbytes in sizes:
        n = nbytes // 4
        t_nccl = torch.ones(n, device="cuda")
        t_p2p = heap.alloc((n,), torch.float32)
        t_p2p.fill_(1.0)
        res = {"bench": "all_reduce_fp32", "bytes": nbytes,
               "nccl_us": timed(lambda: dist.all_reduce(t_nccl)),
               "peer_push_us": timed(lambda: collectives.all_reduce(t_p2p, multicast=False))}
        if heap.multicast_base():
            t_mc = heap.alloc((n,), torch.float32)
            t_mc.fill_(1.0)
            res["multimem_us"] = timed(lambda: collectives.all_reduce(t_mc, multicast=True))
        # bus bandwidth as NCCL defines it: 2 (P-1)/P bytes per byte reduced
        best = min(v for k, v in res.items() if k.endswith("_us") and k != "nccl_us")
        res["busbw_gbs_best"] = round(2 * (world - 1) / world * nbytes / best / 1e3, 1)
        res["busbw_gbs_nccl"] = round(2 * (world - 1) / world * nbytes / res["nccl_us"] / 1e3, 1)
        emit(**{k: (round(v, 1) if isinstance(v, float) else v) for k, v in res.items()})
    for nbytes in (256 << 10, 4 << 20, 32 << 20):
        n = nbytes // 4 // world * world
        a_in, a_out = torch.ones(n, device="cuda"), torch.empty(n, device="cuda")
        h_in, h_out = heap.alloc((n,), torch.float32), heap.alloc((n,), torch.float32)
        h_in.fill_(1.0)
        emit(bench="all_to_all_fp32", bytes=n * 4,
             nccl_us=round(timed(lambda: dist.all_to_all_single(a_out, a_in)), 1),
             peer_push_us=round(timed(lambda: collectives.all_to_all(h_in, h_out)), 1))
    # overlap efficiency: 16 MB all-reduce next to a 4096^3 bf16 GEMM on a second stream
    nbytes = 16 << 20
    g_nccl = torch.ones(nbytes // 4, device="cuda")
    g_ours = heap.alloc((nbytes // 4,), torch.float32)
    a = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(4096, 4096, device="cuda", dtype=torch.bfloat16)
    side = torch.cuda.Stream()

    def overlapped(comm, compute):
        def fn():
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                comm()
            compute()
        return fn

    for name, comm, compute in (("nccl+cublas", lambda: dist.all_reduce(g_nccl), lambda: torch.mm(a, w.t(), out=out)),
                                ("maco_b200", lambda: collectives.all_reduce(g_ours), lambda: ops.gemm(a, w, out=out, max_ctas=116))):
        t_comm, t_comp = timed(comm), timed(compute)
        t_both = timed(overlapped(comm, compute), streams=(side,))
        emit(bench="overlap_efficiency", arm=name, comm_us=round(t_comm, 1), compute_us=round(t_comp, 1),
             overlapped_us=round(t_both, 1), efficiency_pct=round(100 * (t_comm + t_comp - t_both) / min(t_comm, t_comp), 1),
             speedup=round((t_comm + t_comp) / t_both, 2))
    assert _native.status() == 0
    if args.out and rank == 0:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    maco.cleanup()


if __name__ == "__main__":
    main()
