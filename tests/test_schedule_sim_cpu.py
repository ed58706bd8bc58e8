"""Static schedules checked on the host: the program builder runs in planning mode (CPU tensors, no tensor maps),
the queues come from the same assignment the kernel gets, and ``simulate_static_queues`` runs them under the
kernel's rules (head of the queue only, both wait conditions, two-CTA halves together, peer signals). A schedule
whose order can deadlock fails here, on any machine, instead of running into a device-side wait budget."""
import pytest
import torch

from maco_b200.ops import megakernel as mk


@pytest.fixture
def planning():
    """A builder on a CPU device plans only: tasks and their order, no tensor maps, no build()."""
    return None


def _bf(*shape):
    return torch.empty(*shape, dtype=torch.bfloat16)


@pytest.mark.parametrize("pair", [False, True])
def test_chain_of_gemms_with_row_events_and_joins_runs_to_completion(planning, pair):
    """Two dependent GEMMs whose second one carries an extra condition: every pair tile has three wait conditions, so
    join tasks appear; they must sit on their consumer's worker, directly in front of it."""
    b = mk.ProgramBuilder(torch.device("cpu"), num_workers=20, cta_pair=pair)
    x, w1, h, w2, y = _bf(1024, 512), _bf(768, 512), _bf(1024, 768), _bf(512, 768), _bf(1024, 512)
    gate = b.new_event()
    b.add_task(int(mk.TaskType.NOP), b"", signals=[gate])
    other = b.new_event()
    b.add_task(int(mk.TaskType.NOP), b"", signals=[other])
    e1 = b.gemm(x, w1, h, extra_waits=[(gate, 1, False, False)])
    b.gemm(h, w2, y, a_ready=e1, extra_waits=[(gate, 1, False, False), (other, 1, False, False)])
    queues = mk.assign_static_queues(b.tasks, b.num_workers, b.num_comm_workers)
    joins = [i for i, t in enumerate(b.tasks) if t.get("attach_to") is not None]
    assert joins, "the second GEMM's tiles have three conditions each: joins expected"
    where = {t: (w, k) for w, q in enumerate(queues) for k, t in enumerate(q)}
    for j in joins:
        (wj, kj), (wt, kt) = where[j], where[b.tasks[j]["attach_to"]]
        assert wj == wt and kj < kt and all(b.tasks[queues[wj][k]].get("attach_to") == b.tasks[j]["attach_to"] for k in range(kj, kt))
    assert sorted(t for q in queues for t in q) == list(range(len(b.tasks)))
    mk.simulate_static_queues([(b.tasks, queues)])


def test_a_join_behind_the_leader_half_would_deadlock_and_the_simulator_sees_it(planning):
    """The failure this check exists for: a condition of the second half of a two-CTA tile queued BEHIND the leader half."""
    b = mk.ProgramBuilder(torch.device("cpu"), num_workers=4, cta_pair=True)
    x, w1, y = _bf(256, 128), _bf(256, 128), _bf(256, 256)
    b.gemm(x, w1, y)
    queues = mk.assign_static_queues(b.tasks, b.num_workers, b.num_comm_workers)
    mk.simulate_static_queues([(b.tasks, queues)])                      # the real order is fine
    # hand-made bad order: a join the partner half waits for, placed behind the leader half on the leader's worker
    tasks = [dict(t) for t in b.tasks]
    ev = b.new_event()
    join = dict(type=int(mk.TaskType.NOP), flags=0, node_id=0, wait_event=[-1, -1], wait_count=[0, 0], signal_event=[ev, -1],
                signal_peer=-1, signal_peer_event=-1, raw=b"", worker=None, pair_half=None)
    tasks.append(join)
    partner = next(i for i, t in enumerate(tasks) if t.get("pair_half") == 1)
    tasks[partner]["wait_event"], tasks[partner]["wait_count"] = [ev, -1], [1, 0]
    bad = [list(q) for q in queues]
    leader_q = next(w for w, q in enumerate(bad) if partner - 1 in q)
    bad[leader_q].insert(bad[leader_q].index(partner - 1) + 1, len(tasks) - 1)
    with pytest.raises(RuntimeError, match="deadlocks"):
        mk.simulate_static_queues([(tasks, bad)])


def test_join_is_a_balanced_tree(planning):
    b = mk.ProgramBuilder(torch.device("cpu"), num_workers=8)
    evs = [b.new_event() for _ in range(64)]
    n0 = len(b.tasks)
    out = b.join([(e, 1, False, False) for e in evs])
    assert len(out) == 2 and len(b.tasks) - n0 == 62
    # depth: follow the events back to the leaves
    made = {t["signal_event"][0]: t for t in b.tasks[n0:]}

    def depth(ev):
        t = made.get(ev)
        return 0 if t is None else 1 + max(depth(e) for e in t["wait_event"] if e >= 0)

    assert max(depth(w[0]) for w in out) == 5                            # log2(64) - 1 levels under the two survivors


def _FakeHeap(rank, world, nbytes=1 << 28):
    from maco_b200.parallel.symm_heap import PlanningHeap
    return PlanningHeap(rank, world, nbytes)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("pair", [False, True])
def test_tensor_parallel_mlp_schedules_of_all_ranks_run_together(planning, world, pair):
    """all-gather -> GEMM -> GEMM -> reduce-scatter, one program per rank, all ranks simulated together: every
    cross-rank condition (arrival of gathered rows, of partial tiles, the closing waits) has to resolve."""
    from maco_b200.parallel import fused
    T, H, F = 128 * world * 2, 256, 512 * world
    rows, f_local = T // world, F // world
    programs = []
    for rank in range(world):
        heap = _FakeHeap(rank, world)
        b = mk.ProgramBuilder(torch.device("cpu"), num_workers=24, num_comm_workers=4, heap=heap, cta_pair=pair)
        x_full = heap.alloc((T, H), torch.bfloat16)
        x_shard = x_full[rank * rows:(rank + 1) * rows]
        staging = heap.alloc((world, rows, H), torch.bfloat16)
        w1, h, w2, y = _bf(2 * f_local, H), _bf(T, f_local), _bf(H, f_local), _bf(rows, H)
        fence = fused.epoch_fence_event(b)
        ag = fused.allgather_push(b, x_shard, x_full, fence=fence)
        order = fused.gathered_order(rank, world, rows // mk.BM, False)
        e1 = b.gemm(x_full, w1, h, epilogue="swiglu", a_ready=ag, m_blocks=order)
        _, e_out = fused.gemm_reduce_scatter(b, h, w2, staging, y, a_ready=e1)
        fused.epoch_fence_signal(b, [(e_out.all_event[0], e_out.all_event[1], False, False)])
        programs.append((b.tasks, mk.assign_static_queues(b.tasks, b.num_workers, b.num_comm_workers)))
    # every rank emits the same events in the same order, so an event index means the same thing everywhere
    assert len({len(t) for t, _ in programs}) == 1
    mk.simulate_static_queues(programs)


def _programs(make, world):
    progs = []
    for rank in range(world):
        heap = _FakeHeap(rank, world, nbytes=1 << 29) if world > 1 else None
        m = make(rank, world, heap)
        builders = getattr(m, "builders", None) or [m.builder]
        b = builders[0]
        progs.append((b.tasks, mk.assign_static_queues(b.tasks, b.num_workers, b.num_comm_workers)))
    return progs


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_model_programs_have_deadlock_free_static_schedules(planning, world):
    """The four layer programs of the package, planned on the CPU for every rank of a 1-8 rank job and run together by
    the schedule simulator: tensor-parallel MLP, data-parallel backward with tile-wise gradient all-reduce, the Qwen3
    decode layer with fused all-reduces, the expert-parallel MoE layer (counted tiles all treated as live)."""
    from maco_b200.models.dp_mlp_stack import DPMLPStackBackward
    from maco_b200.models.moe_layer import MoEEPLayer
    from maco_b200.models.qwen3_layer import Qwen3DecodeLayer
    from maco_b200.models.tp_mlp import TPSwiGLUMLP
    cpu = torch.device("cpu")
    mk.simulate_static_queues(_programs(
        lambda r, w, h: TPSwiGLUMLP(256 * w, 256, 512 * w, rank=r, world=w, heap=h, device=cpu, num_workers=24, comm_workers=4), world))
    mk.simulate_static_queues(_programs(
        lambda r, w, h: DPMLPStackBackward(layers=3, hidden=max(512, 128 * w), tokens=512, rank=r, world=w, heap=h, device=cpu,
                                           comm_workers=4), world))
    mk.simulate_static_queues(_programs(
        lambda r, w, h: Qwen3DecodeLayer(hidden=1024, q_heads=8 * max(2, w), kv_heads=max(2, w), ffn=2048, batch=8, kv_len=300,
                                         rank=r, world=w, heap=h, device=cpu), world))
    mk.simulate_static_queues(_programs(
        lambda r, w, h: MoEEPLayer(hidden=256, experts=8, top_k=2, inter=128, tokens=256, rank=r, world=w,
                                   heap=h if h is not None else _FakeHeap(0, 1), device=cpu, capacity_factor=4.0), world))


def test_split_k_finishing_form_follows_the_destination(planning):
    """A local result is finished by the last-arriving tile (no SPLITK_FIN tasks); a result that goes into every rank's
    heap keeps the finishing tasks (spread over all workers)."""
    b = mk.ProgramBuilder(torch.device("cpu"), num_workers=32)
    x, w, out = _bf(64, 1024), _bf(512, 1024), _bf(64, 512)
    ev = b.gemm_splitk(x, w, out, split_k=4)
    kinds = [t["type"] for t in b.tasks]
    assert mk.T_SPLITK_FIN not in kinds and kinds.count(int(mk.TaskType.LINEAR)) == 2 * 4
    assert ev.all_event[1] == 8                                     # every tile signals; the last arrival has finished the columns
    b2 = mk.ProgramBuilder(torch.device("cpu"), num_workers=32, heap=_FakeHeap(0, 2))
    arrived = b2.new_event()
    ev2 = b2.gemm_splitk(x, w, None, split_k=4, heap_out_off=4096, ld_out=512, signal_peer_event=arrived)
    kinds2 = [t["type"] for t in b2.tasks]
    assert kinds2.count(mk.T_SPLITK_FIN) == ev2.all_event[1] > 0
    assert all(t["signal_peer"] == -2 for t in b2.tasks if t["type"] == mk.T_SPLITK_FIN)
    # blocked weights: shape is checked
    from maco_b200.ops.gemm import block_weight
    b.gemm_splitk(x, w, out, split_k=4, w_blocked=block_weight(w))
    with pytest.raises(ValueError, match="w_blocked"):
        b.gemm_splitk(x, w, out, split_k=4, w_blocked=w)


def test_several_slot_residual_epilogue_packs_and_validates(planning):
    import struct
    b = mk.ProgramBuilder(torch.device("cpu"), num_workers=8)
    i = b.add_epilogue(0x1000, 512, torch.bfloat16, 256, 512, mode="residual", aux_ptr=0x2000, ld_aux=512, aux_dtype=torch.bfloat16,
                       aux_slots=(4, 1, 256))
    pack = struct.unpack_from("<i", b.epis[i], len(b.epis[i]) - 4)[0]
    assert pack & 15 == 4 and (pack >> 4) & 15 == 1 and pack >> 8 == 256
    with pytest.raises(ValueError):
        b.add_epilogue(0x1000, 512, torch.bfloat16, 256, 512, mode="residual", aux_ptr=0x2000, ld_aux=512,
                       aux_dtype=torch.bfloat16, aux_slots=(1, 0, 256))
    j = b.add_epilogue(0, 256, torch.bfloat16, 512, 256, mode="scatter_rows", aux_ptr=0x3000, bias_type=8)
    mode, _, bias_type = struct.unpack_from("<iii", b.epis[j], 40)
    assert mode == mk.EPI["scatter_rows"] and bias_type == 8


def test_qk_rope_finishing_checks_its_tensors(planning):
    """The QKV projection that finishes with QK-norm + RoPE + cache scatter: shapes are validated when the program is planned."""
    b = mk.ProgramBuilder(torch.device("cpu"), num_workers=32)
    B, hq, hkv, S = 8, 6, 2, 33
    x, w = _bf(B, 512), _bf((hq + 2 * hkv) * 128, 512)
    rope = dict(q_out=_bf(B, hq, 128), k_cache=_bf(B, hkv, S, 128), v_cache=_bf(B, hkv, S, 128), q_norm=_bf(128), k_norm=_bf(128),
                cos_sin=_bf(B, 128), hq=hq, hkv=hkv, pos=S - 1, eps=1e-6)
    ev = b.gemm_splitk(x, w, None, epilogue="qk_rope", rope=rope, split_k=2)
    assert mk.T_SPLITK_FIN not in [t["type"] for t in b.tasks] and ev.all_event[1] == 2 * (hq + 2 * hkv) // 2
    with pytest.raises(ValueError, match="qk_rope"):
        b.gemm_splitk(x, w, _bf(B, (hq + 2 * hkv) * 128), epilogue="qk_rope", rope=rope)           # no output buffer in this form
    with pytest.raises(ValueError, match="rope tensors"):
        b.gemm_splitk(x, w, None, epilogue="qk_rope", rope=dict(rope, pos=S))                      # outside the cache
    with pytest.raises(ValueError, match="rope tensors"):
        b.gemm_splitk(x, w, None, epilogue="qk_rope", rope=dict(rope, hq=hq + 1))                  # heads do not match the weight


def test_makespan_estimate_orders_and_accounts(planning):
    """The timed run of the schedules: a chain of dependent tasks costs the sum of its durations plus one hop per edge,
    independent tasks on different workers overlap, and more communication workers finish an all-gather earlier."""
    b = mk.ProgramBuilder(torch.device("cpu"), num_workers=4)
    e1, e2 = b.new_event(), b.new_event()
    b.add_task(int(mk.TaskType.NOP), b"", signals=[e1])
    b.add_task(int(mk.TaskType.NOP), b"", waits=[(e1, 1, False, False)], signals=[e2])
    b.add_task(int(mk.TaskType.NOP), b"", waits=[(e2, 1, False, False)])
    b.add_task(int(mk.TaskType.NOP), b"")                                   # independent, on another worker
    q = mk.assign_static_queues(b.tasks, b.num_workers, 0)
    r = mk.estimate_makespan([(b.tasks, q)], cost=lambda t: 10.0, hop_us=2.0)
    assert r["span_us"][0] == pytest.approx(3 * 10.0 + 2 * 2.0)
    assert 0 < r["busy_fraction"][0] <= 1

    from maco_b200.models.tp_mlp import TPSwiGLUMLP
    ends = []
    for cw in (2, 8):
        progs = []
        for rank in range(4):
            m = TPSwiGLUMLP(2048, 512, 2048, rank=rank, world=4, heap=_FakeHeap(rank, 4), device=torch.device("cpu"),
                            num_workers=32, comm_workers=cw)
            bb = m.builders[0]
            progs.append((bb.tasks, mk.assign_static_queues(bb.tasks, bb.num_workers, bb.num_comm_workers)))
        res = mk.estimate_makespan(progs)
        assert len(set(round(s, 3) for s in res["span_us"])) == 1            # symmetric ranks end together
        ends.append(res["last_end_by_type_us"][0][int(mk.TaskType.ALLGATHER)])
    assert ends[1] < ends[0]
