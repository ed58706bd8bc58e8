"""The persistent task kernel: static and dynamic scheduling, tile-level dependencies, tracing,
and the bounded-wait failure path (a wait that nothing satisfies returns a status; nothing hangs)."""
import pytest
import torch

import maco_b200 as maco
from maco_b200 import _native
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu


def _mlp_program(mode, tokens=1024, hidden=1024, ffn=2048, workers=None, trace=False, cta_pair=False):
    from maco_b200.ops import interleave_gate_up, megakernel as mk
    dt = torch.bfloat16
    x = torch.randn(tokens, hidden, device="cuda", dtype=dt)
    nw = torch.randn(hidden, device="cuda", dtype=dt)
    wg = torch.randn(ffn, hidden, device="cuda", dtype=dt) * 0.03
    wu = torch.randn(ffn, hidden, device="cuda", dtype=dt) * 0.03
    wd = torch.randn(hidden, ffn, device="cuda", dtype=dt) * 0.03
    wgu = interleave_gate_up(wg, wu)
    xn = torch.empty_like(x)
    h = torch.empty(tokens, ffn, device="cuda", dtype=dt)
    y = torch.empty(tokens, hidden, device="cuda", dtype=dt)
    b = mk.ProgramBuilder(torch.device("cuda"), num_workers=workers, mode=mode, trace=trace, cta_pair=cta_pair)
    e0 = b.elementwise(104, x, xn, in1=nw, rows=tokens, cols=hidden, f0=1e-6)
    e1 = b.gemm(xn, wgu, h, epilogue="swiglu", a_ready=e0)
    b.gemm(h, wd, y, epilogue="residual", aux=x, a_ready=e1)
    prog = b.build()
    xf = x.float()
    nf = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()).to(dt).float()
    hf = (torch.nn.functional.silu(nf @ wg.float().t()) * (nf @ wu.float().t())).to(dt).float()
    ref = hf @ wd.float().t() + xf
    return prog, y, ref


@pytest.mark.parametrize("mode", ["static", "dynamic"])
@pytest.mark.parametrize("workers", [None, 5])
def test_fused_mlp_program(mode, workers):
    prog, y, ref = _mlp_program(mode, workers=workers)
    for _ in range(3):                      # re-execution: events are monotonic, nothing is reset
        y.zero_()
        prog.run()
    torch.cuda.synchronize()
    assert _native.status() == 0
    assert_close(y, ref, torch.bfloat16)
    assert prog.tasks_completed() == 3 * prog.num_tasks
    assert "tile tasks" in prog.describe()


@pytest.mark.parametrize("tokens", [1024, 640, 2304])
@pytest.mark.parametrize("workers", [None, 6])
def test_fused_mlp_program_two_cta_tiles(tokens, workers):
    """The same program on two-CTA tiles (cluster launch, cta_group::2): whole pairs of row blocks, an odd block
    count (one pair gets a filler half), a ragged last block, few and many worker pairs, re-execution."""
    prog, y, ref = _mlp_program("static", tokens=tokens, workers=workers, cta_pair=True)
    assert prog.cta_pair and prog.num_workers % 2 == 0
    for _ in range(3):
        y.zero_()
        prog.run()
    torch.cuda.synchronize()
    assert _native.status() == 0
    assert_close(y, ref, torch.bfloat16)
    assert "two-CTA" in prog.describe()


def test_two_cta_tiles_with_joined_wait_conditions():
    """Tiles with three wait conditions get join tasks; in a two-CTA program the joins of both halves must precede
    both halves in the queues (few workers, so every queue holds joins and halves of many tiles)."""
    from maco_b200.ops import megakernel as mk
    dt = torch.bfloat16
    x = torch.randn(1024, 512, device="cuda", dtype=dt)
    s1, s2 = torch.randn(256, 512, device="cuda", dtype=dt), torch.randn(256, 512, device="cuda", dtype=dt)
    w = torch.randn(768, 512, device="cuda", dtype=dt) * 0.05
    xn, o1, o2 = torch.empty_like(x), torch.empty_like(s1), torch.empty_like(s2)
    y = torch.empty(1024, 768, device="cuda", dtype=dt)
    b = mk.ProgramBuilder(torch.device("cuda"), num_workers=6, cta_pair=True)
    e0 = b.elementwise(112, x, xn, rows=1024, cols=512, f0=2.0)                     # scale: row-block events
    ea = b.elementwise(105, s1, o1, rows=256, cols=512)
    eb = b.elementwise(106, s2, o2, rows=256, cols=512)
    b.gemm(xn, w, y, a_ready=e0, extra_waits=[(ea.all_event[0], ea.all_event[1], False, False),
                                               (eb.all_event[0], eb.all_event[1], False, False)])
    prog = b.build()
    for _ in range(3):
        y.zero_()
        prog.run()
    torch.cuda.synchronize()
    assert _native.status() == 0
    assert_close(y, (2.0 * x.float()).to(dt).float() @ w.float().t(), dt)


def test_two_cta_program_backward_majors():
    """dgrad (plain a @ b: MN-major B) and wgrad (a^T @ b: both operands MN-major) as two-CTA tiles in one program."""
    from maco_b200.ops import megakernel as mk
    dt = torch.bfloat16
    T, H = 1024, 768
    dy = torch.randn(T, H, device="cuda", dtype=dt)
    w = torch.randn(H, H, device="cuda", dtype=dt) * 0.05
    xin = torch.randn(T, H, device="cuda", dtype=dt)
    dx = torch.empty(T, H, device="cuda", dtype=dt)
    dw = torch.empty(H, H, device="cuda", dtype=torch.float32)
    b = mk.ProgramBuilder(torch.device("cuda"), cta_pair=True)
    b.gemm(dy, w, dx, trans_b=True)                                   # dx = dy @ w
    b.gemm(dy, xin, dw, trans_a=True, trans_b=True, epilogue="f32")   # dw = dy^T @ x
    prog = b.build()
    for _ in range(2):
        prog.run()
    torch.cuda.synchronize()
    assert _native.status() == 0
    assert_close(dx, dy.float() @ w.float(), dt)
    torch.testing.assert_close(dw, dy.float().t() @ xin.float(), atol=0.3, rtol=2e-2)


@pytest.mark.parametrize("cta_pair", [False, True])
def test_fused_mlp_program_is_bitwise_deterministic(cta_pair):
    """Five launches of the same program on the same inputs give bit-identical outputs (tile order may differ
    between launches; every output element is still produced by one tile with a fixed accumulation order)."""
    prog, y, _ = _mlp_program("static", cta_pair=cta_pair)
    outs = []
    for _ in range(5):
        y.zero_()
        prog.run()
        torch.cuda.synchronize()
        outs.append(y.clone())
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    assert _native.status() == 0


def test_trace_and_stats():
    prog, y, ref = _mlp_program("static", trace=True)
    prog.run()
    torch.cuda.synchronize()
    st = prog.stats()
    assert st["tasks"] == prog.num_tasks and "LINEAR" in st["by_type"] and "RMSNORM" in st["by_type"]
    ev = prog.chrome_trace()
    assert len(ev) == prog.num_tasks and all(e["dur"] >= 0 for e in ev)


@pytest.mark.parametrize("mode", ["static", "dynamic"])
def test_unsatisfied_wait_times_out_and_context_survives(mode):
    """A task that waits on an event nothing signals: the kernel gives up after its budget, reports
    TIMEOUT with the task and event, returns normally, and the device stays usable."""
    from maco_b200.ops import megakernel as mk
    x = torch.randn(256, 256, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(x)
    b = mk.ProgramBuilder(torch.device("cuda"), num_workers=4, mode=mode, wait_budget_ms=20.0)
    orphan = b.new_event()
    b.elementwise(105, x, out, rows=256, cols=256, extra_waits=[(orphan, 1, False, False)])
    prog = b.build()
    _native.status(clear=True)
    prog.run()
    torch.cuda.synchronize()                # returns: nothing hangs
    st = _native.status(clear=True)
    assert st & _native.STATUS_TIMEOUT
    assert torch.all(out == 0)              # the blocked task never ran
    prog.reset_after_failure()
    # the context is intact: a normal program runs right after
    prog2, y, ref = _mlp_program("static", tokens=256, hidden=256, ffn=512)
    prog2.run()
    torch.cuda.synchronize()
    assert _native.status() == 0
    assert_close(y, ref, torch.bfloat16)


def test_graph_lowering_modes(monkeypatch):
    for mode in ("static", "dynamic"):
        monkeypatch.setenv("MACO_PERSISTENT_MODE", mode)
        g = maco.TaskGraph()
        x = torch.randn(300, 512, device="cuda", dtype=torch.float16)
        w1 = torch.randn(768, 512, device="cuda", dtype=torch.float16) * 0.05
        w2 = torch.randn(512, 768, device="cuda", dtype=torch.float16) * 0.05
        a = g.linear(x, w1, activation="gelu")
        b = g.linear(a.output, w2)
        c = g.add(b.output, x)
        s = g.softmax(c.output)
        g.compile(runtime="persistent")
        g.execute(); g.execute()
        torch.cuda.synchronize()
        F = torch.nn.functional
        af = F.gelu(x.float() @ w1.float().t(), approximate="tanh").half().float()
        cf = ((af @ w2.float().t()).half().float() + x.float()).half().float()
        assert_close(s.output, torch.softmax(cf, -1), torch.float16)
        assert "Persistent kernel" in g.summary()
    assert _native.status() == 0


def test_sm_scheduling_demo_barrier():
    import ctypes
    lib = _native.lib()
    lib.maco_run_sm_scheduling_demo.restype = ctypes.c_float
    lib.maco_run_sm_scheduling_demo.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                ctypes.c_void_p, ctypes.c_void_p]
    n, ctas, tasks = 1 << 20, 8, 10
    data = torch.ones(n, device="cuda")
    order = torch.zeros(ctas * tasks, dtype=torch.int32, device="cuda")
    ms = lib.maco_run_sm_scheduling_demo(data.data_ptr(), n, ctas, 128, tasks, order.data_ptr(), None)
    assert ms > 0
    ref = torch.ones(1, dtype=torch.float64)
    for _ in range(tasks):
        ref = (ref.float() * 1.5 + 0.1).double()
    torch.testing.assert_close(data, torch.full_like(data, float(ref)), rtol=1e-5, atol=1e-5)
    o = order.cpu().view(tasks, ctas)
    assert all(sorted(row.tolist()) == list(range(ctas)) for row in o)   # every barrier round saw each CTA once
    assert _native.status() == 0


@pytest.mark.parametrize("mode", ["static", "dynamic"])
@pytest.mark.parametrize("epilogue", [None, "swiglu", "residual"])
@pytest.mark.parametrize("fused,blocked", [(True, False), (False, False), (True, True)])
def test_splitk_decode_gemm(mode, epilogue, fused, blocked):
    """Few-row GEMM as split-K tiles with fp32 vector reductions, finished by the tile that arrives last for its
    columns (fused) or by separate finishing tasks, run three times: the finishing pass must leave the workspace
    zeroed (and the arrival counters consistent) for the next launch."""
    from maco_b200.ops import interleave_gate_up, megakernel as mk
    dt = torch.bfloat16
    M, K, Nn = 48, 1536, 1024
    x = torch.randn(M, K, device="cuda", dtype=dt)
    w = torch.randn(Nn, K, device="cuda", dtype=dt) * 0.03
    xf = x.float()
    if epilogue == "swiglu":
        wg, wu = w[: Nn // 2], w[Nn // 2:]
        wk = interleave_gate_up(wg.contiguous(), wu.contiguous(), block=128)
        ref = torch.nn.functional.silu(xf @ wg.float().t()) * (xf @ wu.float().t())
        out = torch.empty(M, Nn // 2, device="cuda", dtype=dt)
        aux = None
    else:
        wk = w
        aux = torch.randn(M, Nn, device="cuda", dtype=dt) if epilogue == "residual" else None
        ref = xf @ w.float().t() + (aux.float() if aux is not None else 0)
        out = torch.empty(M, Nn, device="cuda", dtype=dt)
    b = mk.ProgramBuilder(torch.device("cuda"), mode=mode)
    from maco_b200.ops import block_weight
    b.gemm_splitk(x, wk, out, split_k=5, epilogue=epilogue, aux=aux, fused_finish=fused,
                  w_blocked=block_weight(wk) if blocked else None)      # tile-by-tile copy of the weight: contiguous boxes
    prog = b.build()
    for _ in range(3):
        out.zero_()
        prog.run()
    torch.cuda.synchronize()
    assert _native.status() == 0
    assert_close(out, ref, dt)


def test_attention_decode_node_multi_chunk():
    """Tensor-core decode attention node: ragged last chunk, several chunks per split (the K/V ring
    wraps), a split whose first scores are far below later ones (the lazy softmax reference has to move)."""
    from maco_b200.ops import megakernel as mk
    dt = torch.bfloat16
    B, hq, hkv, S, kv_len = 3, 16, 2, 1100, 1037
    q = torch.randn(B, hq, 128, device="cuda", dtype=dt)
    k = torch.randn(B, hkv, S, 128, device="cuda", dtype=dt)
    v = torch.randn(B, hkv, S, 128, device="cuda", dtype=dt)
    k[:, :, 600:640] *= 4.0                       # a late burst of large scores
    out = torch.empty_like(q)
    b = mk.ProgramBuilder(torch.device("cuda"))
    b.attention_decode(q, k, v, out, kv_len=kv_len, splits=2)
    prog = b.build()
    for _ in range(2):
        out.zero_()
        prog.run()
    torch.cuda.synchronize()
    assert _native.status() == 0
    G = hq // hkv
    p = torch.softmax(torch.einsum("bhgd,bhsd->bhgs", q.float().view(B, hkv, G, 128), k[:, :, :kv_len].float()) * 128 ** -0.5, -1)
    ref = torch.einsum("bhgs,bhsd->bhgd", p, v[:, :, :kv_len].float()).reshape(B, hq, 128)
    assert_close(out, ref, dt)
