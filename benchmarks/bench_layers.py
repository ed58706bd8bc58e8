#!/usr/bin/env python
"""Device-timed latency of the target layer configurations, this package vs the library path.

    python benchmarks/bench_layers.py --config {tp_mlp,dp_backward,qwen3_decode} --gpus N [--steps K --warmup W]
    (N > 1: starts one rank per GPU with torch.distributed.run on 127.0.0.1)

"ours" is one launch of the persistent kernel per step. "library" is the same math as separate
launches of the kernels the reference's live runtime calls (torch.mm / cuBLAS, torch element-wise
ops, torch.distributed / NCCL collectives), with the reference's two-stream overlap where it
offers one. Times are CUDA events around K steps, max over ranks; rank 0 prints one JSON line per arm
with the achieved fraction of the roofline (slower of FLOPs / measured GEMM peak and bytes / bandwidth).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def peaks():
    p = {"bf16_tflops_sustained": 1400.0, "bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}
    try:
        d = json.load(open(os.path.join(REPO, "MEASURED_PEAKS.json")))
        p.update({k: d[k] for k in ("bf16_tflops_sustained", "bf16_tflops", "hbm_gbs") if k in d})
        p["source"] = "measured"
    except Exception:
        pass
    # per direction per GPU: the peer-copy rate measured on this pool (the rooflines use it); 900 GB/s is nominal
    p["nvlink_gbs"] = 770.0
    p["nvlink_gbs_nominal"] = 900.0
    return p


def timed(torch, dist, world, steps, fn):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms * 1e3 / steps


# ---------------------------------------------------------------------------------------------------
# configurations: each returns (step_ours, step_library, roofline dict)
# ---------------------------------------------------------------------------------------------------
def cfg_tp_mlp(torch, dist, rank, world, heap, args):
    from maco_b200.models.tp_mlp import TPSwiGLUMLP
    T, H, F = 8192, 4096, 14336
    layer = TPSwiGLUMLP(T, H, F, rank=rank, world=world, heap=heap, mode=args.mode, trace=args.trace)
    args.program = layer.program
    layer.x_shard.normal_()
    rows = T // world
    x_shard = layer.x_shard.clone()
    x_full = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    y_shard = torch.empty(rows, H, device="cuda", dtype=torch.bfloat16)

    def library():
        if world > 1:
            dist.all_gather_into_tensor(x_full, x_shard)
        else:
            x_full.copy_(x_shard)
        h = torch.nn.functional.silu(x_full @ layer.w_gate.t()) * (x_full @ layer.w_up.t())
        y = h @ layer.w_down.t()
        if world > 1:
            dist.reduce_scatter_tensor(y_shard, y)

    # the same layer written against the public TaskGraph API (arm "graph"): allgather -> linear(swiglu) -> linear ->
    # reduce_scatter, lowered to one persistent launch
    import maco_b200 as maco
    from maco_b200 import ops
    gr = maco.TaskGraph()
    if world > 1:
        # the shard is this rank's slice of the gathered buffer (both in the symmetric heap): no local copy
        x_all = heap.alloc((T, H), torch.bfloat16)
        xs_g = x_all[rank * rows:(rank + 1) * rows]
        xs_g.copy_(x_shard)
        ag = gr.allgather(xs_g, output=x_all)
        hh = gr.linear(ag.output, layer.w_gate_up, activation="swiglu")
        yy = gr.linear(hh.output, layer.w_down)
        gr.reduce_scatter(yy.output)
    else:
        hh = gr.linear(x_shard, layer.w_gate_up, activation="swiglu")
        gr.linear(hh.output, layer.w_down)
    from maco_b200.config import config as _cfg
    _cfg.set(profile=bool(args.trace))
    gr.compile()
    _cfg.set(profile=False)
    args.graph_program = getattr(gr._runtime, "_program", None)
    args.graph_step = gr.execute
    args.graph_kind = gr.runtime_kind
    p = peaks()
    flops = 2.0 * T * H * F * 3 / world
    link = (T * H * 2) * (world - 1) / world                       # bytes in (all-gather) = bytes out (partials)
    roof = {"compute_us": flops / (p["bf16_tflops_sustained"] * 1e12) * 1e6, "nvlink_us": link / (p["nvlink_gbs"] * 1e9) * 1e6}
    return (lambda: layer.forward(None)), library, roof


def cfg_dp_backward(torch, dist, rank, world, heap, args):
    from maco_b200.models.dp_mlp_stack import DPMLPStackBackward
    L, H, T = args.layers, 4096, 8192
    m = DPMLPStackBackward(L, H, T, rank=rank, world=world, heap=heap, mode=args.mode, trace=args.trace,
                           cta_pair=bool(args.cta_pair))
    args.program = m.program
    m.forward()
    grads = [torch.empty(H, H, device="cuda", dtype=torch.float32) for _ in range(L)]
    comm = torch.cuda.Stream()
    F = torch.nn.functional

    def gelu_grad(z):
        zf = z.float()
        k0, k1 = 0.7978845608028654, 0.044715
        t = torch.tanh(k0 * (zf + k1 * zf ** 3))
        return 0.5 * (1 + t) + 0.5 * zf * (1 - t * t) * k0 * (1 + 3 * k1 * zf * zf)

    def library():
        # the reference's overlap pattern: backward GEMMs on the compute stream, each layer's fp32
        # gradient all-reduce on a second stream behind an event
        cur = torch.cuda.current_stream()
        dz = ((m.a[-1].float() - m.target.float()) * (2.0 / (T * H)) * gelu_grad(m.z[-1])).to(torch.bfloat16)
        for l in range(L - 1, -1, -1):
            inp = m.a[l - 1] if l > 0 else m.x
            grads[l].copy_((dz.t() @ inp).float() / world)
            if world > 1:
                ev = torch.cuda.Event(); ev.record(cur)
                comm.wait_event(ev)
                with torch.cuda.stream(comm):
                    dist.all_reduce(grads[l])
            if l > 0:
                dz = ((dz @ m.weights[l]).float() * gelu_grad(m.z[l - 1])).to(torch.bfloat16)
        cur.wait_stream(comm)

    p = peaks()
    flops = m.flops()
    link = L * H * H * 4 * 2.0 * (world - 1) / world               # two-shot all-reduce: reduce-scatter + all-gather
    roof = {"compute_us": flops / (p["bf16_tflops_sustained"] * 1e12) * 1e6, "nvlink_us": link / (p["nvlink_gbs"] * 1e9) * 1e6}
    return m.backward, library, roof


def cfg_qwen3_decode(torch, dist, rank, world, heap, args):
    from maco_b200.models.qwen3_layer import Qwen3DecodeLayer
    layer = Qwen3DecodeLayer(rank=rank, world=world, heap=heap, mode=args.mode, trace=args.trace)
    args.program = layer.program
    layer.x.normal_()
    F = torch.nn.functional
    B, D, hq, hkv, G = layer.batch, layer.D, layer.hq, layer.hkv, layer.G
    rms = lambda t, w: (t.float() * torch.rsqrt(t.float().pow(2).mean(-1, keepdim=True) + layer.eps) * w.float()).to(t.dtype)
    cs = layer.cos_sin.float()
    cos, sin = cs[:, : D // 2].unsqueeze(1), cs[:, D // 2:].unsqueeze(1)

    def norm_rope(t, w):
        t = rms(t, w).float()
        t1, t2 = t[..., : D // 2], t[..., D // 2:]
        return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1).to(torch.bfloat16)

    def library():
        x = layer.x
        qkv = rms(x, layer.w_in) @ layer.w_qkv.t()
        q = norm_rope(qkv[:, : hq * D].view(B, hq, D), layer.q_norm)
        k = norm_rope(qkv[:, hq * D:(hq + hkv) * D].view(B, hkv, D), layer.k_norm)
        layer.k_cache[:, :, layer.pos] = k
        layer.v_cache[:, :, layer.pos] = qkv[:, (hq + hkv) * D:].view(B, hkv, D)
        a = F.scaled_dot_product_attention(q.view(B, hkv, G, D), layer.k_cache, layer.v_cache).reshape(B, hq * D)
        o = a @ layer.w_o.t()
        if world > 1:
            dist.all_reduce(o)
        y1 = o + x
        h2 = rms(y1, layer.w_post)
        act = F.silu(h2 @ layer.w_gate.t()) * (h2 @ layer.w_up.t())
        d = act @ layer.w_down.t()
        if world > 1:
            dist.all_reduce(d)
        return d + y1

    p = peaks()
    roof = {"hbm_us": layer.bytes_streamed() / (p["hbm_gbs"] * 1e9) * 1e6,
            "compute_us": 2.0 * B * sum(t.numel() for t in (layer.w_qkv, layer.w_o, layer.w_gate_up, layer.w_down)) / (p["bf16_tflops_sustained"] * 1e12) * 1e6}
    return (lambda: layer.forward(None)), library, roof


def cfg_moe(torch, dist, rank, world, heap, args):
    from maco_b200.models.moe_layer import MoEEPLayer
    H, E, K, I, T = 2048, 128, 8, 768, 4096
    layer = MoEEPLayer(H, E, K, I, T, rank=rank, world=world, heap=heap if world > 1 else None, mode=args.mode, trace=args.trace)
    args.program = layer.program
    layer.x.normal_()
    F = torch.nn.functional
    EL = E // world
    wg, wu, wd = torch.stack(layer.w_gate), torch.stack(layer.w_up), torch.stack(layer.w_down)

    def library():
        # the usual library formulation: top-k, sort by expert, variable-split all-to-all, per-expert GEMMs, return
        x = layer.x
        val, idx = torch.topk(x @ layer.w_router.t(), K, dim=-1)
        w = torch.softmax(val.float(), -1)
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        send = x[order // K]
        counts = torch.bincount(flat, minlength=E)
        if world > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts)
            in_splits = counts.view(world, EL).sum(1).tolist()
            out_splits = recv_counts.view(world, EL).sum(1).tolist()
            recv = torch.empty(sum(out_splits), H, device=x.device, dtype=x.dtype)
            dist.all_to_all_single(recv, send, out_splits, in_splits)
            per = recv_counts.view(world, EL)
        else:
            recv, per, in_splits, out_splits = send, counts.view(1, EL), None, None
        # rows arrive grouped by source rank, then by expert: walk the (source, expert) segments
        out_rows = torch.empty_like(recv)
        seg = per.reshape(-1).tolist()
        pos = 0
        for i, n in enumerate(seg):
            if n:
                el = i % EL
                xs = recv[pos:pos + n]
                out_rows[pos:pos + n] = (F.silu(xs @ wg[el].t()) * (xs @ wu[el].t())) @ wd[el].t()
            pos += n
        if world > 1:
            back = torch.empty_like(send)
            dist.all_to_all_single(back, out_rows, in_splits, out_splits)
        else:
            back = out_rows
        res = torch.zeros(T, H, device=x.device, dtype=torch.float32)
        res.index_add_(0, order // K, back.float() * w.reshape(-1)[order].unsqueeze(1))
        return res.to(x.dtype)

    p = peaks()
    flops = T * K * 2.0 * (3 * H * I) + 2.0 * T * H * E
    link = T * K * H * 2 * (world - 1) / world
    roof = {"compute_us": flops / (p["bf16_tflops_sustained"] * 1e12) * 1e6, "nvlink_us": 2 * link / (p["nvlink_gbs"] * 1e9) * 1e6}
    return (lambda: layer.forward(None)), library, roof


CONFIGS = {"tp_mlp": cfg_tp_mlp, "dp_backward": cfg_dp_backward, "qwen3_decode": cfg_qwen3_decode, "moe": cfg_moe}
HEAP_MB = {"tp_mlp": 512, "dp_backward": 2500, "qwen3_decode": 64, "moe": 700}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=sorted(CONFIGS))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--mode", default="static", choices=["static", "dynamic"])
    ap.add_argument("--arms", default="library,ours")
    ap.add_argument("--cta-pair", type=int, default=1, choices=[0, 1], help="two-CTA GEMM tiles where the model offers them")
    ap.add_argument("--impl", default="", choices=["", "reference"],
                    help="reference: run the unmodified reference package through its own API instead "
                         "(benchmarks/bench_layers_reference.py; tp_mlp: bench.py --impl reference)")
    ap.add_argument("--trace-file", default="", help="with --trace: write the Chrome-trace JSON of rank 0 here")
    ap.add_argument("--trace", action="store_true", help="record the device task trace of one step and print per-type statistics")
    args = ap.parse_args()
    if args.impl == "reference":
        script = os.path.join(REPO, "bench.py") if args.config == "tp_mlp" else os.path.join(REPO, "benchmarks", "bench_layers_reference.py")
        extra = ["--impl", "reference"] if args.config == "tp_mlp" else ["--config", args.config, "--layers", str(args.layers)]
        sys.exit(subprocess.call([sys.executable, script, "--gpus", str(args.gpus), "--steps", str(args.steps),
                                  "--warmup", str(args.warmup)] + extra))
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    real_stdout = os.dup(1)
    os.dup2(2, 1)                         # native libraries print banners on fd 1
    import torch
    import torch.distributed as dist
    rank, local_rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local_rank)
    import maco_b200 as maco
    from maco_b200 import _native
    from maco_b200.parallel import symm_heap
    heap = None
    if world > 1:
        maco.config.set(comm_buffer_size=f"{HEAP_MB[args.config]}MB", backend="peer")
        maco.init(backend="nccl")
        heap = symm_heap.current_heap()
    ours, library, roof = CONFIGS[args.config](torch, dist, rank, world, heap, args)
    p = peaks()
    bound = max(roof.values())
    arms = [("library", library), ("ours", ours)]
    if getattr(args, "graph_step", None) is not None:
        arms.append(("graph", args.graph_step))
    for arm, fn in arms:
        if arm not in args.arms.split(","):
            continue
        for _ in range(args.warmup):
            fn()
        us = timed(torch, dist, world, args.steps, fn)
        if rank == 0:
            line = {"config": args.config, "impl": arm, "n_gpus": world, "latency_us": round(us, 2), "steps": args.steps,
                    "warmup": args.warmup, "roofline_us": {k: round(v, 1) for k, v in roof.items()},
                    "fraction_of_roofline": round(bound / us, 3), "peaks": p["source"],
                    "nvlink_gbs": {"measured_used": p["nvlink_gbs"], "nominal": p["nvlink_gbs_nominal"]},
                    "kernel_status": _native.status(clear=False)}
            if arm == "graph":
                line["runtime"] = args.graph_kind
            os.write(real_stdout, (json.dumps(line) + "\n").encode())
            if arm == "graph" and args.trace and getattr(args, "graph_program", None) is not None:
                os.write(real_stdout, (json.dumps({"config": args.config, "graph_trace": args.graph_program.stats()}) + "\n").encode())
            if arm == "ours" and args.trace:
                os.write(real_stdout, (json.dumps({"config": args.config, "trace": args.program.stats()}) + "\n").encode())
                if args.trace_file:
                    with open(args.trace_file, "w") as f:        # Chrome-trace events, one row per SM
                        json.dump(args.program.chrome_trace(), f)
    if world > 1:
        maco.cleanup()


if __name__ == "__main__":
    main()
