"""Peer-memory collectives and the fused multi-GPU layers, one process per GPU, on every world size in
{2, 4, 8} that the machine has GPUs for."""
import pytest
import torch

from tests._dist import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

ENV = {"NCCL_NVLS_ENABLE": "0"}


def _env(heap_mode):
    """MACO_HEAP: "nvls" = the symmetric heap bound to an NVSwitch multicast object (multimem tasks on; a box whose GPUs
    cannot join one runs it as plain peer memory), "ipc" = the CUDA-IPC form without the binding."""
    return dict(ENV, MACO_HEAP=heap_mode)
_NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
worlds = pytest.mark.parametrize("world", [pytest.param(w, marks=pytest.mark.skipif(_NGPU < w, reason=f"needs {w} GPUs"))
                                           for w in (2, 4, 8)])
# (world, heap form) pairs: the multicast-bound heap at every size, the IPC form (the fallback where a GPU cannot join
# a multicast object) at two ranks; MACO_TEST_ALL_HEAPS=1 adds the IPC form at four and eight
import os as _os
_PAIRS = [(2, "nvls"), (2, "ipc"), (4, "nvls"), (8, "nvls")] + ([(4, "ipc"), (8, "ipc")] if _os.environ.get("MACO_TEST_ALL_HEAPS") == "1" else [])
world_heaps = pytest.mark.parametrize("world,heap_mode", [
    pytest.param(w, h, id=f"{w}-{h}", marks=pytest.mark.skipif(_NGPU < w, reason=f"needs {w} GPUs")) for w, h in _PAIRS])


def _setup(rank, world, heap_mb=256):
    import maco_b200 as maco
    maco.config.set(comm_buffer_size=f"{heap_mb}MB", backend="peer")
    maco.init(backend="nccl")
    from maco_b200.parallel import symm_heap
    return maco, symm_heap.current_heap()


def _collectives(rank, world):
    maco, heap = _setup(rank, world)
    from maco_b200 import _native
    from maco_b200.parallel import collectives
    assert heap is not None and heap.world == world and maco.is_nvshmem_available()
    import os
    assert heap.mode in ("nvls", "vmm", "ipc") and (os.environ["MACO_HEAP"] != "ipc" or heap.mode == "ipc")
    # all-reduce, closed form P(P+1)/2; repeated to exercise the epoch logic
    for dtype, n in ((torch.float32, 1 << 20), (torch.bfloat16, 3 << 16)):
        t = heap.alloc((n,), dtype)
        for it in range(3):
            t.fill_(float(rank + 1))
            collectives.all_reduce(t)
            torch.cuda.synchronize()
            assert torch.all(t.float() == world * (world + 1) / 2), (dtype, it)
    t = heap.alloc((4096,), torch.float32)
    t.fill_(float(rank + 1))
    collectives.all_reduce(t, avg=True)
    torch.cuda.synchronize()
    assert torch.allclose(t, torch.full_like(t, (world + 1) / 2))
    # through the public patterns API and the nvshmem-compatible names
    from maco_b200.comm import patterns
    u = heap.alloc((1000 * 8,), torch.float32)
    u.fill_(float(rank))
    patterns.allreduce(u)
    torch.cuda.synchronize()
    assert torch.all(u == sum(range(world)))
    v = torch.full((333,), float(rank + 1), device="cuda")          # outside the heap, odd size
    maco.nvshmem_allreduce(v)
    torch.cuda.synchronize()
    assert torch.all(v == world * (world + 1) / 2)
    maco.nvshmem_barrier()
    # the multimem forms against the peer-memory forms on the same data (only on a multicast-bound heap)
    if heap.multicast_base():
        g = torch.Generator(device="cuda").manual_seed(5 + rank)
        data = torch.randn(1 << 18, device="cuda", generator=g)
        for dtype in (torch.float32, torch.bfloat16, torch.float16):
            a_mc, a_p2p = heap.alloc((1 << 18,), dtype), heap.alloc((1 << 18,), dtype)
            a_mc.copy_(data)
            a_p2p.copy_(data)
            collectives.all_reduce(a_mc, multicast=True)
            collectives.all_reduce(a_p2p, multicast=False)
            torch.cuda.synchronize()
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert torch.allclose(a_mc.float(), a_p2p.float(), atol=tol * world, rtol=tol), dtype
        sh = heap.alloc((256, 512), torch.bfloat16)
        sh.copy_(data[: 256 * 512].view(256, 512))
        f_mc, f_p2p = heap.alloc((256 * world, 512), torch.bfloat16), heap.alloc((256 * world, 512), torch.bfloat16)
        from maco_b200.parallel import fused
        from maco_b200.ops.megakernel import ProgramBuilder
        for full, mc in ((f_mc, True), (f_p2p, False)):
            b = ProgramBuilder(heap.device, num_workers=8, heap=heap)
            ready = collectives._open(b)
            ev = fused.allgather_push(b, sh, full, fence=ready, multicast=mc)
            collectives._wait_local(b, [(e_, c_, True, False) for e_, c_ in ev.row_events if c_])
            prog = b.build()
            for _ in range(2):
                prog.run()
            torch.cuda.synchronize()
        assert torch.equal(f_mc, f_p2p)
    # all-gather
    shard = heap.alloc((256, 512), torch.bfloat16)
    full = heap.alloc((256 * world, 512), torch.bfloat16)
    shard.fill_(float(rank + 1))
    collectives.all_gather(shard, full)
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.all(full[r * 256:(r + 1) * 256].float() == r + 1)
    # 4-D Ulysses exchange, value-checked, and its inverse
    B, s, H, D = 2, 8, 4 * world, 64
    whole = torch.arange(B * s * world * H * D, dtype=torch.float32, device="cuda").reshape(B, s * world, H, D)
    mine = heap.alloc((B, s, H, D), torch.float32)
    mine.copy_(whole[:, rank * s:(rank + 1) * s])
    y = collectives.all_to_all_4d(mine, 2, 1)
    torch.cuda.synchronize()
    hp = H // world
    assert torch.equal(y, whole[:, :, rank * hp:(rank + 1) * hp])
    z = collectives.all_to_all_4d(y, 1, 2)
    torch.cuda.synchronize()
    assert torch.equal(z, mine)
    # run twice + round trip on random data: identical bits every time
    rnd = heap.alloc((B, s, H, D), torch.bfloat16)
    rnd.copy_(torch.randn(B, s, H, D, device="cuda"))
    first = collectives.all_to_all_4d(rnd, 2, 1).clone()
    for _ in range(4):
        again = collectives.all_to_all_4d(rnd, 2, 1)
        torch.cuda.synchronize()
        assert torch.equal(first, again)
    back = collectives.all_to_all_4d(again, 1, 2)
    torch.cuda.synchronize()
    assert torch.equal(back, rnd)
    # q, k, v back to back through the public call: three results, none overwritten by a later exchange
    qkv = [heap.alloc((B, s, H, D), torch.float32) for _ in range(3)]
    for i, t_ in enumerate(qkv):
        t_.copy_(whole[:, rank * s:(rank + 1) * s] * (i + 1))
    outs = [patterns.all_to_all_4D(t_, 2, 1) for t_ in qkv]
    torch.cuda.synchronize()
    for i, o_ in enumerate(outs):
        assert torch.equal(o_, whole[:, :, rank * hp:(rank + 1) * hp] * (i + 1)), i
    # the same input three times through the low-level call: a result survives the next call on that input
    r1 = collectives.all_to_all_4d(qkv[0], 2, 1)
    qkv[0].mul_(2)
    r2 = collectives.all_to_all_4d(qkv[0], 2, 1)
    torch.cuda.synchronize()
    assert torch.equal(r1, whole[:, :, rank * hp:(rank + 1) * hp]) and torch.equal(r2, 2 * whole[:, :, rank * hp:(rank + 1) * hp])
    # caller-provided destination
    dest = heap.alloc((B, s * world, hp, D), torch.float32)
    assert collectives.all_to_all_4d(qkv[1], 2, 1, out=dest) is dest
    torch.cuda.synchronize()
    assert torch.equal(dest, 2 * whole[:, :, rank * hp:(rank + 1) * hp])
    # broadcast from rank 1, repeated (the receive counter only grows)
    bt = heap.alloc((3 << 18,), torch.float32)
    for it in range(2):
        bt.fill_(float(100 * rank + it))
        collectives.broadcast(bt, src=1)
        torch.cuda.synchronize()
        assert torch.all(bt == 100 + it), it
    # reduce-scatter: block r of the sum ends up on rank r
    rin = heap.alloc((world * 512, 256), torch.bfloat16)
    rout = heap.alloc((512, 256), torch.bfloat16)
    for blk in range(world):
        rin[blk * 512:(blk + 1) * 512].fill_(float((rank + 1) * (blk + 1)))
    collectives.reduce_scatter(rin, rout)
    torch.cuda.synchronize()
    assert torch.all(rout.float() == (rank + 1) * world * (world + 1) / 2)
    # all-to-all with equal and with variable splits (all_to_all_single semantics)
    ain = heap.alloc((world * 64, 128), torch.float32)
    aout = heap.alloc((world * 64, 128), torch.float32)
    for d in range(world):
        ain[d * 64:(d + 1) * 64].fill_(float(10 * rank + d))
    collectives.all_to_all(ain, aout)
    torch.cuda.synchronize()
    for s_ in range(world):
        assert torch.all(aout[s_ * 64:(s_ + 1) * 64] == 10 * s_ + rank)
    in_splits = [8 * (1 + (rank + d) % 3) for d in range(world)]            # what I send to d
    out_splits = [8 * (1 + (s_ + rank) % 3) for s_ in range(world)]         # what s sends to me
    vin = heap.alloc((24 * world, 64), torch.float32)[: sum(in_splits)]      # same allocation on every rank
    vout = heap.alloc((24 * world, 64), torch.float32)[: sum(out_splits)]
    o = 0
    for d in range(world):
        vin[o:o + in_splits[d]].fill_(float(10 * rank + d))
        o += in_splits[d]
    vout.fill_(-1.0)
    torch.cuda.synchronize()
    maco.nvshmem_barrier()            # a peer's rows must not land before this rank has finished clearing vout
    collectives.all_to_all(vin, vout, in_splits, out_splits)
    torch.cuda.synchronize()
    o = 0
    for s_ in range(world):
        assert torch.all(vout[o:o + out_splits[s_]] == 10 * s_ + rank)
        o += out_splits[s_]
    # point-to-point put + flag around the ring
    ps = heap.alloc((1 << 16,), torch.float32)
    pr = heap.alloc((1 << 16,), torch.float32)
    ps.fill_(float(rank + 7))
    collectives.send_recv(ps, (rank + 1) % world, pr, (rank - 1) % world)
    torch.cuda.synchronize()
    assert torch.all(pr == (rank - 1) % world + 7)
    assert _native.status() == 0
    maco.cleanup()


@world_heaps
def test_peer_collectives(world, heap_mode):
    run_ranks(_collectives, world, env=_env(heap_mode), timeout=150)


def _tp_mlp(rank, world):
    maco, heap = _setup(rank, world, heap_mb=128)
    import torch.distributed as dist
    from maco_b200 import _native
    from maco_b200.models.tp_mlp import TPSwiGLUMLP
    tokens, hidden, ffn = 1024, 1024, 2048
    layer = TPSwiGLUMLP(tokens, hidden, ffn, rank=rank, world=world, heap=heap, seed=3, input_slots=2)
    torch.manual_seed(7)
    x_full = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)      # same on every rank
    rows = tokens // world
    partial = layer.reference(x_full)
    dist.all_reduce(partial)
    ref = partial[rank * rows:(rank + 1) * rows]
    outs = []
    for it in range(5):
        y = layer(x_full[rank * rows:(rank + 1) * rows], slot=it & 1)       # alternating input slots
        torch.cuda.synchronize()
        err = (y.float() - ref).abs().max().item()
        assert err < 3e-2 * max(1.0, ref.abs().max().item()), (it, err)
        outs.append(y.clone())
    # repeated runs are bit-identical: partial tiles are summed slot by slot in a fixed order
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    assert _native.status() == 0
    maco.cleanup()


@world_heaps
def test_fused_tp_mlp_matches_reference(world, heap_mode):
    run_ranks(_tp_mlp, world, env=_env(heap_mode), timeout=150)


@pytest.mark.skipif(_NGPU < 4, reason="needs 4 GPUs")
def test_fused_tp_mlp_with_the_reduction_in_the_own_tiles_epilogue_at_four_ranks():
    """Four ranks, own tiles of the GEMM -> reduce-scatter add the three peer slots in their epilogue (the several-slot
    residual epilogue; the default above two ranks is reduction tasks)."""
    env = _env("nvls")
    env["MACO_EPILOGUE_REDUCE_MAX_WORLD"] = "4"
    run_ranks(_tp_mlp, 4, env=env, timeout=150)


def _dp_backward(rank, world):
    maco, heap = _setup(rank, world, heap_mb=192)
    import torch.distributed as dist
    from maco_b200 import _native
    from maco_b200.models.dp_mlp_stack import DPMLPStackBackward
    # a 128-row block of every gradient is owned by one rank: hidden / 128 has to be a multiple of the world size
    m = DPMLPStackBackward(layers=3, hidden=max(512, 128 * world), tokens=1024, rank=rank, world=world, heap=heap, seed=5,
                           weight_std=0.05, comm_workers=4)
    ref = m.reference_grads()
    dist.all_reduce(ref)
    ref /= world
    for it in range(2):
        m.forward()
        grads = m.backward()
        torch.cuda.synchronize()
        err = (grads - ref).abs().max().item()
        assert err < 3e-2 * ref.abs().max().item() + 1e-7, (it, err, ref.abs().max().item())
    assert _native.status() == 0
    maco.cleanup()


@worlds
def test_dp_backward_with_tilewise_allreduce(world):
    run_ranks(_dp_backward, world, env=ENV, timeout=150)


def _qwen3(rank, world):
    maco, heap = _setup(rank, world, heap_mb=64)
    import torch.distributed as dist
    from maco_b200 import _native
    from maco_b200.models.qwen3_layer import Qwen3DecodeLayer
    layer = Qwen3DecodeLayer(hidden=1024, q_heads=8 * max(2, world), kv_heads=max(2, world), ffn=2048, batch=8, kv_len=300, rank=rank, world=world,
                             heap=heap, seed=4, weight_std=0.05)
    torch.manual_seed(11)
    x = torch.randn(8, 1024, device="cuda", dtype=torch.bfloat16)        # replicated input

    def ar(t):
        t = t.clone()
        dist.all_reduce(t)
        return t

    ref = layer.reference(x, ar)
    for it in range(3):
        out = layer(x)
        torch.cuda.synchronize()
        err = (out.float() - ref).abs().max().item()
        assert err < 4e-2 * max(1.0, ref.abs().max().item()), (it, err)
    assert _native.status() == 0
    maco.cleanup()


@worlds
def test_qwen3_decode_layer_tensor_parallel(world):
    run_ranks(_qwen3, world, env=ENV, timeout=150)


def _moe(rank, world):
    maco, heap = _setup(rank, world, heap_mb=64)
    from maco_b200 import _native
    from maco_b200.models.moe_layer import MoEEPLayer
    layer = MoEEPLayer(hidden=256, experts=8, top_k=2, inter=128, tokens=256, rank=rank, world=world, heap=heap,
                       capacity_factor=4.0, seed=3, weight_std=0.05, router_std=0.5)
    torch.manual_seed(100 + rank)
    x = torch.randn(256, 256, device="cuda", dtype=torch.bfloat16)          # every rank has its own tokens
    ref = layer.reference(x)
    for it in range(3):
        out = layer(x)
        torch.cuda.synchronize()
        assert layer.dropped() == 0
        err = (out.float() - ref).abs().max().item()
        assert err < 4e-2 * max(1.0, ref.abs().max().item()), (it, err)
    assert _native.status() == 0
    maco.cleanup()


@worlds
def test_moe_expert_parallel_dispatch_combine(world):
    run_ranks(_moe, world, env=ENV, timeout=150)


def _peer_loss(rank, world):
    """Rank 1 leaves between steps with nothing in flight; rank 0 learns of it on the host (heartbeat in
    the rendezvous store) before its next launch, raises PeerLostError and shuts down without collectives."""
    import os
    maco, heap = _setup(rank, world, heap_mb=32)
    from maco_b200 import PeerLostError, _native
    from maco_b200.comm.process_group import ProcessGroupManager, ensure_peers
    from maco_b200.parallel import collectives
    t = heap.alloc((1 << 16,), torch.float32)
    for step in (1, 2):
        ensure_peers(step, timeout_s=20.0)
        t.fill_(float(rank + 1))
        collectives.all_reduce(t)
        torch.cuda.synchronize()
        assert torch.all(t == world * (world + 1) / 2)
    pgm = ProcessGroupManager()
    if rank == 1:
        pgm.heartbeat(2)
        pgm.announce_exit()
        torch.cuda.synchronize()
        os._exit(0)                       # gone; no kernel or collective of this rank is in flight
    lost = None
    try:
        ensure_peers(3, timeout_s=10.0)
    except PeerLostError as exc:
        lost = exc.rank
    assert lost == 1
    assert _native.status() == 0
    maco.cleanup(abort=True)
    os._exit(0)


def test_peer_loss_detected_before_the_next_launch():
    # plain peer memory: a rank must not leave while its heap is bound to a multicast object
    run_ranks(_peer_loss, 2, env=_env("ipc"), timeout=100)


def _graph_collectives(rank, world):
    """Multi-rank TaskGraphs run inside ONE launch of the persistent kernel: all-gather -> GEMM, GEMM ->
    reduce-scatter, all-reduce, all-to-all and broadcast nodes, with tensors inside and outside the heap."""
    maco, heap = _setup(rank, world, heap_mb=256)
    import torch.distributed as dist
    from maco_b200 import _native, ops
    dt = torch.bfloat16
    F = torch.nn.functional
    tokens, hidden, ffn = 128 * world * 2, 512, 1024
    rows = tokens // world
    torch.manual_seed(3)
    x_full = torch.randn(tokens, hidden, device="cuda", dtype=dt)                  # same on every rank
    g = torch.Generator(device="cuda").manual_seed(10 + rank)
    wg = torch.randn(ffn // world, hidden, device="cuda", dtype=dt, generator=g) * 0.05
    wu = torch.randn(ffn // world, hidden, device="cuda", dtype=dt, generator=g) * 0.05
    wd = torch.randn(hidden, ffn // world, device="cuda", dtype=dt, generator=g) * 0.05
    for in_heap in (True, False):
        x_shard = heap.alloc((rows, hidden), dt) if in_heap else torch.empty(rows, hidden, device="cuda", dtype=dt)
        x_shard.copy_(x_full[rank * rows:(rank + 1) * rows])
        gr = maco.TaskGraph()
        ag = gr.allgather(x_shard)
        h = gr.linear(ag.output, ops.interleave_gate_up(wg, wu), activation="swiglu")
        y = gr.linear(h.output, wd)
        rs = gr.reduce_scatter(y.output)
        gr.compile()
        assert gr.runtime_kind == "persistent", gr.runtime_kind
        hf = (F.silu(x_full.float() @ wg.float().t()) * (x_full.float() @ wu.float().t())).to(dt).float()
        part = hf @ wd.float().t()
        dist.all_reduce(part)
        ref = part[rank * rows:(rank + 1) * rows]
        for it in range(3):
            gr.execute()
            torch.cuda.synchronize()
            assert torch.equal(ag.output, x_full), (in_heap, it)
            err = (rs.output.float() - ref).abs().max().item()
            assert err < 3e-2 * max(1.0, ref.abs().max().item()), (in_heap, it, err)
    # all-reduce (sum and avg, inside and outside the heap), broadcast, flat and 4-D all-to-all in one graph
    gr = maco.TaskGraph()
    a_h = heap.alloc((1 << 16,), torch.float32)
    a_o = torch.empty(3000, device="cuda", dtype=torch.float32)                    # 12000 bytes: a multiple of 16
    bc = heap.alloc((4096,), torch.float32)
    flat = torch.empty(world * 64, 32, device="cuda", dtype=torch.float32)
    B, s, H, D = 2, 8, 4 * world, 64
    whole = torch.arange(B * s * world * H * D, dtype=torch.float32, device="cuda").reshape(B, s * world, H, D)
    q4 = torch.empty(B, s, H, D, device="cuda", dtype=torch.float32)
    n1 = gr.allreduce(a_h)
    n2 = gr.allreduce(a_o, op="avg")
    n3 = gr.broadcast(bc, src=world - 1)
    n4 = gr.all_to_all(flat, scatter_dim=0, gather_dim=0)
    n5 = gr.all_to_all(q4, scatter_dim=2, gather_dim=1)
    n6 = gr.all_to_all(n5.output, scatter_dim=1, gather_dim=2)
    gr.compile()
    assert gr.runtime_kind == "persistent", gr.runtime_kind
    hp = H // world
    for it in range(3):
        a_h.fill_(float(rank + 1 + it))
        a_o.fill_(float(rank + it))
        bc.fill_(float(10 * rank + it))
        for d in range(world):
            flat[d * 64:(d + 1) * 64].fill_(float(100 * rank + d + it))
        q4.copy_(whole[:, rank * s:(rank + 1) * s] + it)
        gr.execute()
        torch.cuda.synchronize()
        assert torch.all(a_h == sum(r + 1 + it for r in range(world))), it
        assert torch.allclose(a_o, torch.full_like(a_o, sum(r + it for r in range(world)) / world)), it
        assert torch.all(bc == 10 * (world - 1) + it), it
        for s_ in range(world):
            assert torch.all(n4.output[s_ * 64:(s_ + 1) * 64] == 100 * s_ + rank + it), (it, s_)
        assert torch.equal(n5.output, whole[:, :, rank * hp:(rank + 1) * hp] + it), it
        assert torch.equal(n6.output, q4), it
    assert _native.status() == 0
    maco.cleanup()


@world_heaps
def test_multirank_taskgraph_runs_in_the_persistent_kernel(world, heap_mode):
    run_ranks(_graph_collectives, world, env=_env(heap_mode), timeout=150)


def _ulysses(rank, world):
    """Ulysses attention end to end: QKV projections + exchanges and inverse exchange + output projection as two
    persistent-kernel launches on heap tensors, against fp32 attention over the whole sequence."""
    maco, heap = _setup(rank, world, heap_mb=128)
    from maco_b200 import _native
    from maco_b200.models.ulysses_attention import UlyssesAttention
    B, S, H, D, hidden = 2, 128 * world, 4 * world, 64, 512
    layer = UlyssesAttention(B, S, H, D, hidden, rank=rank, world=world, heap=heap, seed=9)
    assert layer.graph_in.runtime_kind == "persistent" and layer.graph_out.runtime_kind == "persistent"
    torch.manual_seed(21)
    x_full = torch.randn(B, S, hidden, device="cuda", dtype=torch.bfloat16)
    s = S // world
    ref = layer.reference(x_full)
    for it in range(3):
        out = layer(x_full[:, rank * s:(rank + 1) * s])
        torch.cuda.synchronize()
        err = (out.float() - ref).abs().max().item()
        assert err < 4e-2 * max(1.0, ref.abs().max().item()), (it, err)
    assert _native.status() == 0
    maco.cleanup()


@worlds
def test_ulysses_attention_on_heap_tensors(world):
    run_ranks(_ulysses, world, env=ENV, timeout=150)
