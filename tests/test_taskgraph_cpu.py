"""TaskGraph front end on CPU: node creation, dependency inference, waves, compile/execute, summary.
Behaviours pinned by the reference's tests/test_taskgraph.py and tests/test_runtime.py."""
import pytest
import torch

import maco_b200 as maco
from maco_b200 import TaskGraph, TaskType


def G(**kw):
    return TaskGraph(num_workers=kw.pop("num_workers", 4), device="cpu", **kw)


def test_empty_graph_compiles_and_executes():
    g = G()
    g.compile()
    g.execute()
    assert len(g) == 0


def test_linear_node_and_output_preallocated():
    g = G()
    x, w = torch.randn(32, 256), torch.randn(512, 256)
    t = g.linear(x, w, name="fc")
    assert t.task_type == TaskType.LINEAR and t.name == "fc"
    assert t.output.shape == (32, 512) and t.is_compute and not t.is_comm
    assert t.dims == [256, 512]


def test_linear_matches_torch_with_bias_and_3d_input():
    g = G()
    x, w, b = torch.randn(4, 8, 64), torch.randn(96, 64), torch.randn(96)
    t = g.linear(x, w, b)
    g.compile(); g.execute()
    torch.testing.assert_close(t.output, torch.nn.functional.linear(x, w, b), atol=1e-5, rtol=1e-5)


def test_user_output_written_in_place():
    g = G()
    x, w = torch.randn(32, 64), torch.randn(48, 64)
    out = torch.zeros(32, 48)
    t = g.linear(x, w, output=out)
    assert t.output is out
    g.execute()
    torch.testing.assert_close(out, x @ w.t(), atol=1e-5, rtol=1e-5)


def test_matmul_and_custom():
    g = G()
    a, b = torch.randn(32, 64), torch.randn(64, 128)
    t = g.matmul(a, b)
    out = torch.empty(32, 128)
    c = g.custom(lambda v: torch.relu(v) * 2, [t.output], [out])
    g.compile()
    assert c.depends_on == [t]
    g.execute()
    torch.testing.assert_close(out, torch.relu(a @ b) * 2, atol=1e-5, rtol=1e-5)


def test_chain_dependencies_and_waves():
    g = G()
    x = torch.randn(16, 32)
    ws = [torch.randn(32, 32) for _ in range(3)]
    cur, tasks = x, []
    for w in ws:
        t = g.linear(cur, w)
        tasks.append(t)
        cur = t.output
    g.compile()
    assert tasks[1].depends_on == [tasks[0]] and tasks[2].depends_on == [tasks[1]]
    assert len(g._schedule.waves) == 3
    assert all(0 <= g._schedule.worker_assignments[t._node_id] < 4 for t in tasks)


def test_independent_tasks_share_a_wave_and_diamond():
    g = G()
    x = torch.randn(8, 16)
    a = g.linear(x, torch.randn(16, 16))
    b = g.linear(x, torch.randn(16, 16))
    s = g.add(a.output, b.output)
    g.compile()
    assert len(g._schedule.waves) == 2 and set(g._schedule.waves[0]) == {a, b}
    assert set(s.depends_on) == {a, b}
    g.execute()
    torch.testing.assert_close(s.output, a.output + b.output)


def test_war_and_waw_hazards_are_ordered():
    g = G()
    x = torch.randn(8, 16)
    buf = torch.empty(8, 16)
    w1 = g.gelu(x, output=buf)          # writes buf
    r = g.silu(buf)                     # reads buf
    w2 = g.scale(x, 2.0, output=buf)    # overwrites buf: must wait for the reader and the first writer
    g.compile()
    assert w1 in r.depends_on and r in w2.depends_on and w1 in w2.depends_on


def test_long_chain_and_reexecute():
    g = G()
    x = torch.randn(4, 32)
    w = torch.eye(32)
    cur = x
    for _ in range(50):
        cur = g.linear(cur, w).output
    g.compile()
    for _ in range(3):
        g.execute()
    torch.testing.assert_close(cur, x)


def test_allreduce_world1_is_noop_and_identity_output():
    g = G()
    x = torch.randn(32, 256)
    before = x.clone()
    t = g.allreduce(x, name="ar")
    g.compile(); g.execute()
    assert t.output is x and t.is_comm
    torch.testing.assert_close(x, before)


def test_all_to_all_world1_copies():
    g = G()
    x = torch.randn(2, 8, 4, 16)
    t = g.all_to_all(x)
    g.execute()
    torch.testing.assert_close(t.output, x)


def test_overlap_roles_and_waves():
    g = G()
    x, w = torch.randn(32, 64), torch.randn(64, 64)
    tasks, cur = [], x
    for _ in range(4):
        t = g.linear(cur, w)
        tasks.append(t)
        cur = t.output
    comm = g.allreduce(torch.randn(32, 64))
    grp = g.overlap(tasks, [comm])
    assert tasks[0]._overlap_role == "compute" and comm._overlap_role == "comm"
    grp.auto_waves()
    assert grp.num_waves == 2
    assert [t._wave_id for t in tasks] == [0, 0, 1, 1]
    grp.with_waves(4)
    assert [t._wave_id for t in tasks] == [0, 1, 2, 3]
    many = g.overlap([g.gelu(x) for _ in range(9)], []).auto_waves()
    assert many.num_waves == 4


def test_untouched_group_gets_auto_waves_at_compile():
    g = G()
    x = torch.randn(8, 8)
    ts = [g.gelu(x) for _ in range(5)]
    grp = g.overlap(ts, [g.allreduce(torch.randn(8))])
    g.compile()
    assert grp.num_waves == 2


def test_summary_strings():
    g = G()
    g.linear(torch.randn(32, 256), torch.randn(512, 256))
    s = g.summary()
    assert "Total nodes: 1" in s and "Compute nodes: 1" in s and "Execution waves" not in s
    g.compile()
    assert "Execution waves" in g.summary()
    assert "TaskGraph(" in repr(g)


def test_builtin_ops_match_torch():
    g = G()
    x = torch.randn(6, 64)
    w, b = torch.randn(64), torch.randn(64)
    nodes = {
        "gelu": g.gelu(x), "silu": g.silu(x), "softmax": g.softmax(x), "rms": g.rmsnorm(x, w, eps=1e-6),
        "ln": g.layernorm(x, w, b), "gate": g.silu_gate(x, x * 0.5), "scale": g.scale(x, 3.0),
    }
    g.execute()
    F = torch.nn.functional
    torch.testing.assert_close(nodes["gelu"].output, F.gelu(x, approximate="tanh"))
    torch.testing.assert_close(nodes["silu"].output, F.silu(x))
    torch.testing.assert_close(nodes["softmax"].output, torch.softmax(x, -1))
    torch.testing.assert_close(nodes["rms"].output, x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w)
    torch.testing.assert_close(nodes["ln"].output, F.layer_norm(x, (64,), w, b), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(nodes["gate"].output, F.silu(x) * x * 0.5)
    torch.testing.assert_close(nodes["scale"].output, x * 3.0)


def test_rope_matches_complex_rotation():
    g = G()
    tokens, heads, hd = 5, 3, 8
    x = torch.randn(tokens, heads, hd)
    ang = torch.randn(tokens, hd // 2)
    t = g.rope(x, ang.cos(), ang.sin())
    g.execute()
    xc = torch.complex(x[..., : hd // 2], x[..., hd // 2:]) * torch.polar(torch.ones_like(ang), ang).unsqueeze(1)
    torch.testing.assert_close(t.output, torch.cat([xc.real, xc.imag], -1), atol=1e-5, rtol=1e-5)


def test_state_dict_roundtrip_keeps_pointers():
    g = G()
    w = torch.randn(16, 16)
    g.register_weight("w", w)
    t = g.linear(torch.randn(4, 16), w)
    g.compile()
    saved = g.state_dict()
    ptr = w.data_ptr()
    w.zero_()
    g.load_state_dict(saved)
    assert w.data_ptr() == ptr and torch.equal(w, saved["w"])
    with pytest.raises(KeyError):
        g.load_state_dict({"other": w})


def test_tasktype_values_match_native_header():
    import re, pathlib
    hdr = (pathlib.Path(maco.__file__).resolve().parent.parent / "csrc" / "maco_types.h").read_text()
    native = {m.group(1): int(m.group(2)) for m in re.finditer(r"MACO_TASK_(\w+)\s*=\s*(\d+)", hdr)}
    for t in TaskType:
        assert native[t.name] == int(t), t
