"""Stream manager, signals, overlap contexts and planners without a GPU (streams are inert
stand-ins), plus SM role configuration, config object, tensor registry and comm scheduler."""
import pytest
import torch

import maco_b200 as maco
from maco_b200 import (CommScheduler, OverlapContext, OverlapMode, OverlapRuntime, OverlapScheduler, Role, SMConfig,
                       SMManager, SignalWait, StreamManager, TensorRegistry, auto_config, create_signal)


def test_stream_manager_singleton_and_reset():
    StreamManager.reset()
    a, b = StreamManager(), StreamManager()
    assert a is b and a.compute_stream is not a.comm_stream
    a.compute_wait_comm(); a.comm_wait_compute(); a.default_wait_all(); a.sync_all()
    StreamManager.reset()
    assert StreamManager() is not a
    assert maco.sync.get_compute_stream() is not None and maco.sync.get_comm_stream() is not None


def test_signal_lifecycle():
    sig = create_signal("s")
    assert sig.name == "s" and not sig.signaled and not sig.is_ready()
    sig.record()
    assert sig.signaled and sig.is_ready()
    sig.wait(); sig.synchronize()


def test_signalwait_named_and_waves():
    sw = SignalWait()
    s = sw.create_signal("compute_done")
    assert sw.get_signal("compute_done") is s
    sw.signal("done"); sw.wait("done")
    with pytest.raises(KeyError):
        sw.wait("missing")
    for i in range(3):
        sw.signal_wave(i)
    assert sw.num_waves == 3
    sw.wait_all_waves()
    sw.reset()
    assert sw.get_signal("done") is None and sw.num_waves == 0


def test_overlap_context_even_odd_waves():
    ctx = OverlapContext()
    results = []
    for w in range(4):
        with ctx.compute():
            results.append(torch.ones(4) * w)
        ctx.signal_compute_done(w)
        with ctx.comm():
            ctx.wait_compute_done(w)
        ctx.signal_comm_done(w)
    ctx.wait_comm_done(3)
    ctx.sync_all()
    assert ctx.signals.num_waves == 8 and len(results) == 4
    assert ctx.signals._waves[6].name == "wave_6" and ctx.signals._waves[7].name == "wave_7"
    ctx.reset()
    assert ctx.signals.num_waves == 0


def test_overlap_plans():
    s = OverlapScheduler()
    comp, comm = list(range(4)), ["c0", "c1"]
    p = s.create_plan(comp, comm, mode=OverlapMode.NONE)
    assert p.mode == OverlapMode.NONE and p.num_waves == 1 and p.compute_waves == [comp]
    p = s.create_plan(comp, comm, mode=OverlapMode.WAVE, num_waves=2)
    assert p.num_waves == 2 and p.compute_waves == [[0, 1], [2, 3]] and p.wave_comm_mapping == {0: ["c0"], 1: ["c1"]}
    p = s.create_plan(list(range(7)), ["a", "b", "c"], mode=OverlapMode.WAVE)
    assert p.num_waves == 3 and sum(len(w) for w in p.compute_waves) == 7


def test_overlap_execution_order():
    trace = []
    rt = OverlapRuntime()
    rt.execute_overlap(list(range(4)), ["c0", "c1"], lambda t: trace.append(("compute", t)),
                       lambda t: trace.append(("comm", t)), mode=OverlapMode.WAVE, num_waves=2)
    assert trace == [("compute", 0), ("compute", 1), ("comm", "c0"), ("compute", 2), ("compute", 3), ("comm", "c1")]
    trace.clear()
    rt.execute_overlap(list(range(2)), ["c0"], lambda t: trace.append(("compute", t)),
                       lambda t: trace.append(("comm", t)), mode=OverlapMode.NONE)
    assert trace == [("compute", 0), ("compute", 1), ("comm", "c0")]


def test_overlap_manager_cpu_fallback():
    maco.init(backend="gloo")
    try:
        t = torch.ones(8)
        res, comm = maco.overlap_compute_and_comm(lambda: torch.arange(4).sum(), t, "allreduce")
        assert int(res) == 6 and torch.equal(comm, torch.ones(8))
        a2a, comp = maco.overlap_all_to_all_with_compute(lambda: t * 2, lambda: 5)
        assert comp == 5 and torch.equal(a2a, torch.full((8,), 2.0))
        with maco.overlap_region() as region:
            f1 = region.comm(lambda: 1)
            f2 = region.compute(lambda: 2)
        assert region.get_comm_results() == [1] and region.get_compute_results() == [2] and f1.wait() == 1 and f2.result() == 2
        assert maco.get_overlap_manager().stats["num_overlaps"] >= 2
        assert maco.get_rank() == 0 and maco.get_world_size() == 1 and maco.is_initialized()
    finally:
        maco.cleanup()
    assert not maco.is_initialized()


def test_sm_config_roles():
    cfg = SMConfig(total_sms=148)
    cfg.assign_role((0, 132), Role.COMPUTE).assign_role((132, 133), Role.LOCAL_SCHEDULER)
    cfg.assign_role((133, 148), Role.REMOTE_SCHEDULER)
    assert (cfg.compute_sms, cfg.local_scheduler_sms, cfg.remote_scheduler_sms) == (132, 1, 15)
    assert cfg.validate() and cfg.to_dict()["total_sms"] == 148
    with pytest.raises(ValueError):
        cfg.assign_role((100, 140), Role.COMPUTE)
    with pytest.raises(ValueError):
        SMConfig(total_sms=8).assign_role((0, 9), Role.COMPUTE)
    with pytest.raises(ValueError):
        SMConfig(total_sms=8).validate()
    c = auto_config("high", "high", total_sms=148)
    assert c.compute_sms == int(148 * 0.70) and c.compute_sms + c.local_scheduler_sms + c.remote_scheduler_sms == 148
    m = SMManager(SMConfig(total_sms=16).assign_role((0, 12), Role.COMPUTE).assign_role((12, 13), Role.LOCAL_SCHEDULER))
    assert m.get_worker_config() == {"num_workers": 12, "num_local_schedulers": 1, "num_remote_schedulers": 0}


def test_config_object():
    cfg = maco.MacoConfig()
    cfg.set(debug=True, comm_buffer_size="64MB")
    assert cfg.get("debug") is True and cfg.comm_buffer_bytes == 64 << 20 and "backend" in cfg.to_dict()
    with pytest.raises(ValueError):
        cfg.set(nonexistent=1)


def test_tensor_registry():
    reg = TensorRegistry()
    w = torch.randn(4, 4)
    reg.register_weight(w, "w"); reg.register_input(torch.randn(2, 4), "x"); reg.register_output((2, 4), "y")
    assert len(reg) == 3 and "w" in reg and reg.get_tensor("w") is w
    assert set(reg.weights) == {"w"} and set(reg.inputs) == {"x"} and set(reg.outputs) == {"y"}
    assert reg.get_all_pointers()["w"] == w.data_ptr()
    with pytest.raises(ValueError):
        reg.register(w, "w")
    reg.clear()
    assert len(reg) == 0


def test_comm_scheduler_phases_and_cycles():
    cs = CommScheduler(num_sms=16)
    g1, g2 = torch.ones(4), torch.ones(4) * 2
    cs.phase("grads").allreduce(g1)
    cs.phase("gather", depends_on=["grads"]).allgather(g2)
    cs.compile()
    info = cs.get_schedule_info()
    assert info["order"] == ["grads", "gather"] and info["num_sms"] == 16
    cs.execute()
    assert cs.phases["gather"].ops[0].result.shape == (1, 4)
    cs.reset()
    cs.phase("a", depends_on=["b"]); cs.phase("b", depends_on=["a"])
    with pytest.raises(ValueError):
        cs.compile()


def test_context_objects():
    with maco.Context(world_size=1) as ctx:
        assert ctx.compute(lambda a: a + 1, 1) == 2
        t = torch.ones(3)
        assert ctx.allreduce(t) is t
    pc = maco.PersistentContext(model=torch.nn.Linear(4, 2), sm_config=SMConfig(total_sms=8).assign_role((0, 8), Role.COMPUTE))
    with pc:
        assert pc(torch.randn(3, 4)).shape == (3, 2)
        pc.register_tensor(torch.randn(2), "t")
        assert pc.worker_config["num_workers"] == 8


def test_host_placement_respects_the_cpus_the_process_may_use(monkeypatch):
    """bind_host_to_gpu only ever narrows the affinity to GPU-local CPUs it is allowed to use, and reports why it
    did nothing otherwise (fake NVML answers; sched_setaffinity is intercepted)."""
    import os
    from maco_b200.utils import numa
    if not hasattr(os, "sched_setaffinity"):
        pytest.skip("no sched_setaffinity")
    allowed = {0, 1, 2, 3}
    calls = []
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(allowed))
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cpus: calls.append(set(cpus)))
    monkeypatch.setattr(numa, "local_cpus", lambda i: {2, 3, 8, 9})
    r = numa.bind_host_to_gpu(0)
    assert r["bound"] and calls == [{2, 3}] and r["cpus"] == 2
    calls.clear()
    monkeypatch.setattr(numa, "local_cpus", lambda i: {8, 9})            # nothing local is available: unchanged
    assert not numa.bind_host_to_gpu(0)["bound"] and calls == []
    monkeypatch.setattr(numa, "local_cpus", lambda i: set())             # NVML knows nothing: unchanged
    assert not numa.bind_host_to_gpu(0)["bound"] and calls == []
    monkeypatch.setattr(numa, "local_cpus", lambda i: {0, 1, 2, 3, 4})   # already local only: unchanged
    assert not numa.bind_host_to_gpu(0)["bound"] and calls == []
    monkeypatch.setenv("MACO_NUMA_BIND", "0")
    monkeypatch.setattr(numa, "local_cpus", lambda i: {2, 3})
    assert not numa.bind_host_to_gpu(0)["bound"] and calls == []
