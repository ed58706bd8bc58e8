"""Collectives and graph communication nodes over gloo with 2 CPU ranks (closed-form checks, the
style of the reference's tests/test_comm.py which needs real GPUs + torchrun)."""
import torch

from tests._dist import run_ranks


def _collectives(rank, world):
    import torch.distributed as dist
    import maco_b200 as maco
    from maco_b200.comm import patterns
    maco.init(backend="gloo")
    assert maco.get_rank() == rank and maco.get_world_size() == world
    pgm = maco.ProcessGroupManager()
    assert pgm.rank == rank and pgm.world_size == world and pgm.is_main_process == (rank == 0)
    # all-reduce: closed form P(P+1)/2, AVG really divides
    t = torch.full((64, 64), float(rank + 1))
    patterns.allreduce(t)
    assert torch.all(t == world * (world + 1) / 2)
    t = torch.full((8,), float(rank + 1))
    patterns.allreduce(t, op=patterns.AVG)
    assert torch.allclose(t, torch.full((8,), (world + 1) / 2))
    h = maco.async_all_reduce(torch.full((4,), float(rank)), async_op=True)
    assert torch.all(h.wait() == sum(range(world))) and h.is_completed()
    # all-gather
    g = patterns.allgather(torch.full((3,), float(rank)))
    assert g.shape == (world, 3) and all(torch.all(g[r] == r) for r in range(world))
    g = maco.async_all_gather(torch.full((2, 3), float(rank))).wait()
    assert g.shape == (2 * world, 3) and torch.all(g[2 * (world - 1)] == world - 1)
    # reduce-scatter
    rs = patterns.reduce_scatter(torch.arange(4 * world, dtype=torch.float32).reshape(2 * world, 2) * (rank + 1))
    full = torch.arange(4 * world, dtype=torch.float32).reshape(2 * world, 2) * (world * (world + 1) / 2)
    assert torch.equal(rs, full.chunk(world, 0)[rank])
    # all-to-all: value src*10 + dst
    send = torch.stack([torch.full((4,), float(rank * 10 + d)) for d in range(world)])
    recv = maco.async_all_to_all(send, scatter_dim=0, gather_dim=0).wait()
    assert all(torch.all(recv[s] == s * 10 + rank) for s in range(world))
    out = patterns.all_to_all_single(None, send.clone())
    assert torch.equal(out, recv)
    # 4-D Ulysses switch and its inverse, value-checked
    B, s, H, D = 2, 3, 2 * world, 4
    full_x = torch.arange(B * s * world * H * D, dtype=torch.float32).reshape(B, s * world, H, D)
    mine = full_x[:, rank * s:(rank + 1) * s]
    y = patterns.all_to_all_4D(mine, 2, 1)
    hp = H // world
    assert torch.equal(y, full_x[:, :, rank * hp:(rank + 1) * hp])
    z = patterns.all_to_all_4D(y, 1, 2)
    assert torch.equal(z, mine)
    assert torch.equal(maco.async_all_to_all_4d(mine, 2, 1).wait(), y)
    # broadcast, send/recv
    b = torch.full((4,), 42.0) if rank == 0 else torch.zeros(4)
    maco.async_broadcast(b, src=0).wait()
    assert torch.all(b == 42)
    if rank == 0:
        patterns.send(torch.full((2,), 7.0), dst=1)
    elif rank == 1:
        assert torch.all(patterns.recv(torch.zeros(2), src=0) == 7)
    maco.comm.barrier()
    maco.cleanup()


def test_collectives_two_ranks():
    run_ranks(_collectives, 2)


def _graph_plumbing(rank, world):
    import maco_b200 as maco
    maco.init(backend="gloo")
    torch.manual_seed(0)
    x = torch.randn(32, 512)
    w1 = torch.randn(1024, 512) / 512 ** 0.5
    w2 = torch.randn(512, 1024) / 1024 ** 0.5
    grad = torch.randn(1 << 20) + rank
    expect_grad = sum(torch.randn_like(grad).copy_(grad - rank + r) for r in range(world))
    g = maco.TaskGraph(num_workers=8)
    t1 = g.linear(x, w1)
    t2 = g.linear(t1.output, w2)
    ar = g.allreduce(grad)
    g.overlap([t1, t2], [ar]).auto_waves()
    avg_in = torch.full((16,), float(rank + 1))
    av = g.allreduce(avg_in, op="avg")
    a2a_in = torch.arange(world * 4, dtype=torch.float32).reshape(world, 4) + 100 * rank
    a2a = g.all_to_all(a2a_in, scatter_dim=0, gather_dim=0)
    ag = g.allgather(torch.full((2, 2), float(rank)))
    rs = g.reduce_scatter(torch.ones(2 * world, 3) * (rank + 1))
    g.compile()
    assert g.runtime_kind == "reference"
    g.execute()
    torch.testing.assert_close(t2.output, (x @ w1.t()) @ w2.t(), atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(grad, expect_grad, atol=1e-5, rtol=1e-5)
    assert torch.allclose(avg_in, torch.full((16,), (world + 1) / 2))
    for s in range(world):
        assert torch.equal(a2a.output[s], torch.arange(4, dtype=torch.float32) + 4 * rank + 100 * s)
    assert ag.output.shape == (2 * world, 2) and torch.all(ag.output[2:4] == 1)
    assert torch.all(rs.output == world * (world + 1) / 2) and rs.output.shape == (2, 3)
    maco.cleanup()


def test_graph_plumbing_two_ranks():
    """Two-linear chain + 1 Mi-element gradient all-reduce with overlap().auto_waves(), world 2."""
    run_ranks(_graph_plumbing, 2)


def _heartbeat(rank, world):
    import time
    import maco_b200 as maco
    maco.init(backend="gloo")
    pgm = maco.ProcessGroupManager()
    pgm.heartbeat(1)
    assert pgm.check_peers(1, timeout_s=10.0) == []
    if rank == 1:
        pgm.announce_exit()          # leaves between steps, nothing in flight
        maco.cleanup()
        return
    lost = pgm.check_peers(2, timeout_s=1.0)
    assert lost == [1], lost
    maco.cleanup()


def test_peer_loss_is_detected_on_the_host():
    run_ranks(_heartbeat, 2)


def _recover(rank, world):
    """Three ranks run two steps; rank 1 leaves between steps with nothing in flight. The two survivors learn of
    it from the heartbeats, tear down without collectives, rendezvous again as a world of two, rebuild their
    graph and all-reduce correctly."""
    import os
    import maco_b200 as maco
    from maco_b200.comm.process_group import ProcessGroupManager, ensure_peers
    maco.init(backend="gloo", timeout_s=30.0)

    def step_graph(value):
        t = torch.full((1024,), float(value))
        g = maco.TaskGraph(num_workers=4)
        ar = g.allreduce(t)
        g.compile()
        g.execute()
        return ar.output

    for step in (1, 2):
        ensure_peers(step, timeout_s=20.0)
        out = step_graph(rank + 1)
        assert torch.all(out == 6.0), (step, out[0])
    pgm = ProcessGroupManager()
    if rank == 1:
        pgm.heartbeat(2)
        pgm.announce_exit()
        os._exit(0)                          # gone: no collective of this rank is in flight
    lost = None
    try:
        ensure_peers(3, timeout_s=5.0)
    except maco.PeerLostError as exc:
        lost = exc.rank
    assert lost == 1
    new_rank, new_world = maco.recover([1], timeout_s=30.0)
    assert new_world == 2 and new_rank == {0: 0, 2: 1}[rank]
    assert maco.get_world_size() == 2 and maco.get_rank() == new_rank
    for step in (1, 2):                      # the recompiled graph runs in the smaller world
        ensure_peers(step, timeout_s=20.0)
        out = step_graph(rank + 1)           # old ranks 0 and 2 contribute 1 + 3
        assert torch.all(out == 4.0), (step, out[0])
    maco.cleanup()
    os._exit(0)


def test_survivors_rerendezvous_and_recompile_after_peer_loss():
    run_ranks(_recover, 3, timeout=120)
