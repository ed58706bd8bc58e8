"""TaskGraph on a GPU: every runtime against PyTorch (tolerances of the reference's tests/test_runtime.py)."""
import pytest
import torch

import maco_b200 as maco
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu


def _runtimes():
    from maco_b200.task_graph.runtime import PersistentRuntime
    kinds = ["stream"]
    try:
        from maco_b200.ops import megakernel  # noqa: F401
        kinds.append("persistent")
    except Exception:
        pass
    return kinds


@pytest.mark.parametrize("kind", ["stream", "persistent"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_linear_chain(kind, dtype):
    if kind not in _runtimes():
        pytest.skip("runtime not built")
    if kind == "persistent" and dtype == torch.float32:
        pytest.skip("the persistent kernel's GEMM tasks are tcgen05 tiles: 16-bit inputs only")
    g = maco.TaskGraph(num_workers=8)
    x = torch.randn(32, 512, device="cuda", dtype=dtype)
    w1 = (torch.randn(1024, 512, device="cuda") / 512 ** 0.5).to(dtype)
    w2 = (torch.randn(512, 1024, device="cuda") / 1024 ** 0.5).to(dtype)
    b1 = torch.randn(1024, device="cuda", dtype=dtype)
    t1 = g.linear(x, w1, b1)
    t2 = g.linear(t1.output, w2)
    g.compile(runtime=kind)
    assert g.runtime_kind == kind
    for _ in range(2):
        g.execute()
    torch.cuda.synchronize()
    ref = torch.nn.functional.linear(torch.nn.functional.linear(x.float(), w1.float(), b1.float()).to(dtype).float(), w2.float())
    assert_close(t2.output, ref, dtype)
    from maco_b200 import _native
    assert _native.status() == 0


@pytest.mark.parametrize("kind", ["stream", "persistent"])
def test_mixed_graph(kind):
    if kind not in _runtimes():
        pytest.skip("runtime not built")
    dt = torch.bfloat16
    g = maco.TaskGraph()
    x = torch.randn(256, 1024, device="cuda", dtype=dt)
    nw = torch.randn(1024, device="cuda", dtype=dt)
    wg = torch.randn(2048, 1024, device="cuda", dtype=dt) * 0.03
    wu = torch.randn(2048, 1024, device="cuda", dtype=dt) * 0.03
    wd = torch.randn(1024, 2048, device="cuda", dtype=dt) * 0.03
    n = g.rmsnorm(x, nw)
    a = g.linear(n.output, wg)
    b = g.linear(n.output, wu)
    s = g.silu_gate(a.output, b.output)
    d = g.linear(s.output, wd)
    r = g.add(d.output, x)
    m = g.matmul(r.output, wg.t().contiguous()[:, :512].contiguous())
    g.compile(runtime=kind)
    g.execute()
    torch.cuda.synchronize()
    F = torch.nn.functional
    xf = x.float()
    nf = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()).to(dt).float()
    sf = (F.silu((nf @ wg.float().t()).to(dt).float()) * (nf @ wu.float().t()).to(dt).float()).to(dt).float()
    rf = ((sf @ wd.float().t()).to(dt).float() + xf).to(dt).float()
    assert_close(r.output, rf, dt)
    assert_close(m.output, rf @ wg.float().t()[:, :512], dt)


def test_custom_node_and_world1_collectives():
    g = maco.TaskGraph(num_workers=4)
    x = torch.randn(32, 256, device="cuda")
    out = torch.empty_like(x)
    c = g.custom(torch.nn.functional.gelu, [x], [out])
    ar = g.allreduce(out)
    a2a = g.all_to_all(torch.randn(2, 4, 8, 16, device="cuda"))
    g.compile(); g.execute()
    torch.cuda.synchronize()
    torch.testing.assert_close(out, torch.nn.functional.gelu(x), atol=1e-5, rtol=1e-5)
    assert ar.output is out and a2a.output.shape == (2, 4, 8, 16)


def test_large_matmul_and_stream_argument():
    g = maco.TaskGraph()
    a = torch.randn(1024, 2048, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(2048, 2048, device="cuda", dtype=torch.bfloat16) * 0.02
    t = g.matmul(a, b)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g.execute(stream=s)
    s.synchronize()
    assert_close(t.output, a.float() @ b.float(), torch.bfloat16)


def test_sync_primitives_on_gpu():
    maco.StreamManager.reset()
    sm = maco.StreamManager()
    assert isinstance(sm.compute_stream, torch.cuda.Stream) and sm.compute_stream is not sm.comm_stream
    ctx = maco.OverlapContext()
    with ctx.compute():
        a = torch.randn(512, 512, device="cuda") @ torch.randn(512, 512, device="cuda")
    ctx.signal_compute_done(0)
    with ctx.comm():
        ctx.wait_compute_done(0)
        c = a.clone()
    ctx.signal_comm_done(0)
    ctx.wait_comm_done(0)
    ctx.sync_all()
    torch.testing.assert_close(a, c)
    sig = maco.create_signal("t")
    assert not sig.is_ready()
    sig.record(); torch.cuda.synchronize()
    assert sig.is_ready()
    res, comm = maco.overlap_compute_and_comm(lambda: a @ a, c, "allreduce")
    torch.cuda.synchronize()
    assert res.shape == (512, 512) and comm is c


def test_decode_shaped_linear_takes_the_split_k_path():
    """A few-row linear with a large weight is lowered to split-K tiles plus finishing tasks; chained with a
    row-wise op and a second linear, executed twice (the partial-sum workspace must come back clean)."""
    g = maco.TaskGraph()
    dt = torch.bfloat16
    x = torch.randn(16, 2048, device="cuda", dtype=dt)
    nw = torch.randn(2048, device="cuda", dtype=dt)
    w1 = (torch.randn(2048, 2048, device="cuda") * 0.03).to(dt)
    w2 = (torch.randn(2304, 2048, device="cuda") * 0.03).to(dt)
    h = g.rmsnorm(x, nw, eps=1e-6)
    t1 = g.linear(h.output, w1)
    t2 = g.linear(t1.output, w2)
    g.compile(runtime="persistent")
    assert g.runtime_kind == "persistent"
    for _ in range(2):
        g.execute()
    torch.cuda.synchronize()
    xf = x.float()
    hf = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()).to(dt).float()
    ref = (hf @ w1.float().t()).to(dt).float() @ w2.float().t()
    assert_close(t2.output, ref, dt)


def test_compiled_schedule_is_cached_for_identical_graphs():
    """Rebuilding the same graph over the same tensors reuses the compiled program; a different shape does not."""
    import maco_b200 as maco
    from maco_b200.task_graph.runtime import PersistentRuntime
    PersistentRuntime.clear_schedule_cache()
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(512, 512, device="cuda", dtype=torch.bfloat16) * 0.05
    out = torch.empty(256, 512, device="cuda", dtype=torch.bfloat16)

    def build(xx):
        g = maco.TaskGraph()
        g.linear(xx, w, output=out if xx is x else None)
        g.compile()
        return g

    g1 = build(x)
    hits = PersistentRuntime.cache_hits
    g2 = build(x)
    assert g1.runtime_kind == g2.runtime_kind == "persistent"
    assert PersistentRuntime.cache_hits == hits + 1 and g2._runtime._program is g1._runtime._program
    g3 = build(torch.randn(384, 512, device="cuda", dtype=torch.bfloat16))
    assert PersistentRuntime.cache_hits == hits + 1 and g3._runtime._program is not g1._runtime._program
    for g in (g1, g2):
        out.zero_()
        g.execute()
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), x.float() @ w.float().t(), atol=1e-1, rtol=5e-2)


def test_persistent_context_compiles_a_sequential_module():
    """PersistentContext turns a chain of supported layers into one persistent-kernel launch per forward."""
    import torch.nn as nn
    from maco_b200.core import PersistentContext, SMConfig, Role
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(512, 1024), nn.GELU(approximate="tanh"), nn.LayerNorm(1024), nn.Linear(1024, 256, bias=False),
                          nn.SiLU()).cuda().to(torch.bfloat16).eval()
    x = torch.randn(384, 512, device="cuda", dtype=torch.bfloat16)
    cfg = SMConfig(total_sms=148)
    cfg.assign_role((0, 96), Role.COMPUTE)
    cfg.assign_role((96, 97), Role.LOCAL_SCHEDULER)
    with torch.no_grad(), PersistentContext(model, cfg) as ctx:
        for _ in range(2):
            y = ctx(x)
            torch.cuda.synchronize()
            assert ctx.last_runtime == "persistent" and ctx.worker_config["num_workers"] == 96
            import copy
            ref = copy.deepcopy(model).float()(x.float())
            torch.testing.assert_close(y.float(), ref, atol=1e-1, rtol=5e-2)
        assert "layer0.weight" in ctx.registry.weights
        # a module the kernel has no tasks for runs as it is
        other = PersistentContext(nn.Sequential(nn.Linear(512, 64), nn.Tanh()).cuda().to(torch.bfloat16))
        other(x)
        assert other.last_runtime == "module"
