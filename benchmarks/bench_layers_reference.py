#!/usr/bin/env python
"""Reference arm of the layer benchmarks: the UNMODIFIED reference package (installed under baseline/_ref) driven
through its own public API, on the same configurations as ``bench_layers.py``.

    python benchmarks/bench_layers_reference.py --config {dp_backward,moe,qwen3_decode} --gpus N [--steps K --warmup W]

What the reference offers and how each configuration uses it:
* GEMMs: ``TaskGraph.linear`` / ``TaskGraph.matmul`` nodes, executed by its ``StreamRuntime`` (torch.mm);
* ops it has no node for (GELU', RMSNorm, RoPE, SiLU-gate, top-k, attention): ``TaskGraph.custom(fn=torch op)``,
  its documented escape hatch (maco/task_graph/runtime.py:228-234);
* collectives: ``TaskGraph.allreduce`` nodes and ``maco.comm.patterns`` (NCCL);
* overlap: ``maco.overlap_compute_and_comm`` (its OverlapManager: compute on one stream, the all-reduce on a second
  one, maco/overlap/manager.py:163-215), used for the data-parallel backward the way its README shows.
None of this package's kernels, models or engine is imported here. Device-timed (CUDA events around K steps), max
over ranks; rank 0 prints one JSON line with ``"impl": "reference"``.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(REPO, "baseline", "_ref")


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


def gelu_grad(torch, z):
    zf = z.float()
    k0, k1 = 0.7978845608028654, 0.044715
    t = torch.tanh(k0 * (zf + k1 * zf ** 3))
    return 0.5 * (1 + t) + 0.5 * zf * (1 - t * t) * k0 * (1 + 3 * k1 * zf * zf)


def ref_dp_backward(torch, dist, maco, rank, world, args):
    """16 x Linear(4096, 4096) + GELU, 8192 tokens per rank: per layer one reference TaskGraph (wgrad matmul, dgrad
    matmul, GELU' as a custom node); the fp32 gradient all-reduce of layer l+1 runs under layer l's graph through
    ``maco.overlap_compute_and_comm``."""
    L, H, T = args.layers, 4096, 8192
    dt = torch.bfloat16
    g = torch.Generator(device="cpu").manual_seed(rank)
    mk = lambda *s, std=1.0: (torch.randn(*s, generator=g) * std).to(dt).cuda()
    weights = [mk(H, H, std=0.02) for _ in range(L)]
    acts = [mk(T, H) for _ in range(L + 1)]              # layer inputs a[l] (a[0] = x); synthetic forward state
    zs = [mk(T, H) for _ in range(L)]                    # pre-activations
    dz = [torch.empty(T, H, device="cuda", dtype=dt) for _ in range(L)]
    grads = [torch.empty(H, H, device="cuda", dtype=torch.float32) for _ in range(L)]
    target = mk(T, H)
    graphs = []
    with contextlib.redirect_stdout(sys.stderr):
        for l in range(L):
            gr = maco.TaskGraph(num_workers=8)
            wg = gr.matmul(dz[l].t(), acts[l], name=f"wgrad{l}")                         # [H, T] @ [T, H]
            gr.custom(lambda w: w.float() / world, [wg.output], [grads[l]], name=f"grad{l}")
            if l > 0:
                dg = gr.matmul(dz[l], weights[l], name=f"dgrad{l}")                      # [T, H] @ [H, H]
                gr.custom(lambda d, z: (d.float() * gelu_grad(torch, z)).to(dt), [dg.output, zs[l - 1]], [dz[l - 1]],
                          name=f"gelu_bwd{l}")
            gr.compile()
            graphs.append(gr)

    def step():
        dz[L - 1].copy_(((acts[L].float() - target.float()) * (2.0 / (T * H)) * gelu_grad(torch, zs[L - 1])).to(dt))
        graphs[L - 1].execute()
        for l in range(L - 2, -1, -1):
            if world > 1:
                maco.overlap_compute_and_comm(graphs[l].execute, grads[l + 1], "allreduce")
            else:
                graphs[l].execute()
        if world > 1:
            maco.comm.patterns.allreduce(grads[0])

    return step


def ref_moe(torch, dist, maco, rank, world, args):
    """MoE expert-parallel layer (hidden 2048, 128 experts, top-8, intermediate 768, 4096 tokens per rank): router
    GEMM as a TaskGraph.linear node, routing / permutation and the per-expert FFNs as custom nodes (the reference
    has no router, top-k or grouped-GEMM node), dispatch and combine through
    ``maco.comm.patterns.all_to_all_single`` with variable splits."""
    H, E, K, I, T = 2048, 128, 8, 768, 4096
    EL = E // world
    dt = torch.bfloat16
    F = torch.nn.functional
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    mk = lambda *s, std=0.02: (torch.randn(*s, generator=g) * std).to(dt).cuda()
    x = mk(T, H, std=1.0)
    w_router = mk(E, H)
    wg, wu, wd = mk(EL, I, H), mk(EL, I, H), mk(EL, H, I)
    patterns = maco.comm.patterns
    state = {}
    with contextlib.redirect_stdout(sys.stderr):
        g1 = maco.TaskGraph(num_workers=8)
        logits = g1.linear(x, w_router, name="router")
        g1.compile()

    def experts(recv, per):
        out_rows = torch.empty_like(recv)
        pos = 0
        for i, n in enumerate(per.reshape(-1).tolist()):       # (source rank, local expert) segments
            if n:
                el = i % EL
                xs = recv[pos:pos + n]
                out_rows[pos:pos + n] = (F.silu(xs @ wg[el].t()) * (xs @ wu[el].t())) @ wd[el].t()
            pos += n
        return out_rows

    def step():
        g1.execute()
        val, idx = torch.topk(logits.output, K, dim=-1)
        w = torch.softmax(val.float(), -1)
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        send = x[order // K]
        counts = torch.bincount(flat, minlength=E)
        if world > 1:
            recv_counts = torch.empty_like(counts)
            patterns.all_to_all_single(recv_counts, counts)
            in_splits = counts.view(world, EL).sum(1).tolist()
            out_splits = recv_counts.view(world, EL).sum(1).tolist()
            recv = torch.empty(sum(out_splits), H, device="cuda", dtype=dt)
            patterns.all_to_all_single(recv, send, out_splits, in_splits)
            per = recv_counts.view(world, EL)
        else:
            recv, per = send, counts.view(1, EL)
        # the expert FFNs through the reference's custom-node mechanism (shapes change every step, so the node is
        # built per step, as its examples do for data-dependent work)
        with contextlib.redirect_stdout(sys.stderr):
            g2 = maco.TaskGraph(num_workers=8)
            out_rows = torch.empty_like(recv)
            g2.custom(lambda r: experts(r, per), [recv], [out_rows], name="experts")
            g2.compile()
            g2.execute()
        if world > 1:
            back = torch.empty_like(send)
            patterns.all_to_all_single(back, out_rows, in_splits, out_splits)
        else:
            back = out_rows
        res = torch.zeros(T, H, device="cuda", dtype=torch.float32)
        res.index_add_(0, order // K, back.float() * w.reshape(-1)[order].unsqueeze(1))
        state["out"] = res.to(dt)

    return step


def ref_qwen3_decode(torch, dist, maco, rank, world, args):
    """Qwen3-32B-shaped decoder layer, decode batch 64, 4096 cached keys, tensor parallel over the ranks: ONE reference
    TaskGraph with linear nodes for the five projections, custom nodes for RMSNorm, QK-norm + RoPE + cache write,
    attention (scaled_dot_product_attention), SiLU-gate and the residual adds, and two allreduce nodes."""
    hidden, hq_all, hkv_all, D, ffn, B, S = 5120, 64, 8, 128, 25600, 64, 4096
    hq, hkv, f_local = hq_all // world, max(1, hkv_all // world), ffn // world
    G = hq // hkv
    dt = torch.bfloat16
    F = torch.nn.functional
    eps, pos = 1e-6, S - 1
    g = torch.Generator(device="cpu").manual_seed(200 + rank)
    mk = lambda *s, std=0.02: (torch.randn(*s, generator=g) * std).to(dt).cuda()
    x = mk(B, hidden, std=1.0)
    w_in, w_post, q_norm, k_norm = (torch.ones(n, device="cuda", dtype=dt) for n in (hidden, hidden, D, D))
    w_qkv, w_o = mk((hq + 2 * hkv) * D, hidden), mk(hidden, hq * D)
    w_gate, w_up, w_down = mk(f_local, hidden), mk(f_local, hidden), mk(hidden, f_local)
    k_cache, v_cache = mk(B, hkv, S, D, std=1.0), mk(B, hkv, S, D, std=1.0)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = (pos * inv).cuda()
    cos, sin = ang.cos().view(1, 1, -1), ang.sin().view(1, 1, -1)
    rms = lambda t, w: (t.float() * torch.rsqrt(t.float().pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(dt)

    def norm_rope(t, w):
        t = rms(t, w).float()
        t1, t2 = t[..., : D // 2], t[..., D // 2:]
        return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1).to(dt)

    def attend(qkv):
        q = norm_rope(qkv[:, : hq * D].view(B, hq, D), q_norm)
        k = norm_rope(qkv[:, hq * D:(hq + hkv) * D].view(B, hkv, D), k_norm)
        k_cache[:, :, pos] = k
        v_cache[:, :, pos] = qkv[:, (hq + hkv) * D:].view(B, hkv, D)
        return F.scaled_dot_product_attention(q.view(B, hkv, G, D), k_cache, v_cache).reshape(B, hq * D)

    buf = lambda *s: torch.empty(*s, device="cuda", dtype=dt)
    xn, att, y1, h2, act, out = buf(B, hidden), buf(B, hq * D), buf(B, hidden), buf(B, hidden), buf(B, f_local), buf(B, hidden)
    with contextlib.redirect_stdout(sys.stderr):
        gr = maco.TaskGraph(num_workers=8)
        gr.custom(lambda t: rms(t, w_in), [x], [xn], name="rmsnorm_in")
        qkv = gr.linear(xn, w_qkv, name="qkv")
        gr.custom(attend, [qkv.output], [att], name="attention")
        o = gr.linear(att, w_o, name="o_proj")
        if world > 1:
            gr.allreduce(o.output, name="ar_attn")
        gr.custom(lambda a, r: a + r, [o.output, x], [y1], name="residual1")
        gr.custom(lambda t: rms(t, w_post), [y1], [h2], name="rmsnorm_post")
        ga = gr.linear(h2, w_gate, name="gate")
        up = gr.linear(h2, w_up, name="up")
        gr.custom(lambda a, b_: F.silu(a) * b_, [ga.output, up.output], [act], name="swiglu")
        dn = gr.linear(act, w_down, name="down")
        if world > 1:
            gr.allreduce(dn.output, name="ar_mlp")
        gr.custom(lambda a, r: a + r, [dn.output, y1], [out], name="residual2")
        gr.compile()
    return gr.execute


CONFIGS = {"dp_backward": ref_dp_backward, "moe": ref_moe, "qwen3_decode": ref_qwen3_decode}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=sorted(CONFIGS))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=16)
    args = ap.parse_args()
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    real_stdout = os.dup(1)
    os.dup2(2, 1)                         # the reference and NCCL print banners on fd 1
    if not os.path.isdir(os.path.join(REF_DIR, "maco")):
        os.write(real_stdout, (json.dumps({"impl": "reference", "unavailable": "baseline/_ref/maco is not installed"}) + "\n").encode())
        return
    import torch
    import torch.distributed as dist
    rank, local_rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local_rank)
    sys.path.insert(0, REF_DIR)
    import maco
    if world > 1:
        maco.init(backend="nccl")
    try:
        step = CONFIGS[args.config](torch, dist, maco, rank, world, args)
        for _ in range(args.warmup):
            step()
        us = timed(torch, dist, world, args.steps, step)
        line = {"config": args.config, "impl": "reference", "n_gpus": world, "latency_us": round(us, 2), "steps": args.steps,
                "warmup": args.warmup, "path": "baseline/_ref maco: TaskGraph + StreamRuntime (torch.mm), custom nodes, "
                                                "maco.comm.patterns / overlap_compute_and_comm (NCCL)"}
    except Exception as exc:                                   # the arm must not take a benchmark run down
        line = {"config": args.config, "impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    if rank == 0:
        os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
