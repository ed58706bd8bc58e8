"""Argument validation and error messages (behaviours pinned by the reference's tests/test_validation.py)."""
import pytest
import torch

from maco_b200 import (AlreadyCompiledError, CyclicDependencyError, DeviceError, DimensionError, DTypeMismatchError,
                       NullInputError, ShapeMismatchError, TaskGraph, TaskGraphError, ValidationError)


def G():
    return TaskGraph(num_workers=4, device="cpu")


def test_none_inputs_name_parameter_and_method():
    g = G()
    w = torch.randn(8, 4)
    with pytest.raises(NullInputError) as e:
        g.linear(None, w)
    assert "input" in str(e.value) and "linear" in str(e.value) and "Hint:" in str(e.value)
    with pytest.raises(NullInputError) as e:
        g.linear(torch.randn(2, 4), None)
    assert "weight" in str(e.value)
    with pytest.raises(NullInputError):
        g.matmul(None, torch.randn(4, 4))
    with pytest.raises(NullInputError):
        g.allreduce(None)
    with pytest.raises(NullInputError):
        g.all_to_all(None)


def test_shape_mismatch_messages_carry_sizes():
    g = G()
    with pytest.raises(ShapeMismatchError) as e:
        g.linear(torch.randn(32, 256), torch.randn(512, 128))
    assert "256" in str(e.value) and "128" in str(e.value)
    with pytest.raises(ShapeMismatchError):
        g.linear(torch.randn(32, 256), torch.randn(512, 256), torch.randn(128))
    with pytest.raises(ShapeMismatchError):
        g.matmul(torch.randn(32, 64), torch.randn(128, 256))
    with pytest.raises(ShapeMismatchError):
        g.linear(torch.randn(4, 8), torch.randn(16, 8), output=torch.empty(4, 15))


def test_dtype_mismatch_names_both_dtypes():
    g = G()
    with pytest.raises(DTypeMismatchError) as e:
        g.linear(torch.randn(4, 8), torch.randn(16, 8, dtype=torch.float16))
    assert "float32" in str(e.value) and "float16" in str(e.value)
    with pytest.raises(DTypeMismatchError):
        g.matmul(torch.randn(4, 8), torch.randn(8, 4, dtype=torch.bfloat16))


def test_dimension_errors():
    g = G()
    with pytest.raises(DimensionError):
        g.linear(torch.randn(4, 8), torch.randn(8))
    with pytest.raises(DimensionError):
        g.matmul(torch.randn(2, 4, 8), torch.randn(8, 4))


def test_custom_needs_callable():
    g = G()
    x = torch.randn(4, 4)
    with pytest.raises(ValidationError) as e:
        g.custom(fn="nope", inputs=[x], outputs=[torch.empty_like(x)])
    assert "callable" in str(e.value).lower()


def test_modify_after_compile_and_idempotent_compile():
    g = G()
    x, w = torch.randn(4, 8), torch.randn(8, 8)
    g.linear(x, w)
    g.compile()
    sched = g._schedule
    g.compile()
    assert g._schedule is sched
    with pytest.raises(AlreadyCompiledError) as e:
        g.linear(x, w)
    assert "Cannot modify" in str(e.value)
    with pytest.raises(AlreadyCompiledError):
        g.allreduce(x)


def test_manual_cycle_is_detected():
    g = G()
    x, w = torch.randn(4, 8), torch.randn(8, 8)
    a = g.linear(x, w, name="a")
    b = g.linear(x, w, name="b")
    c = g.linear(x, w, name="c")
    a.add_dependency(c); b.add_dependency(a); c.add_dependency(b)
    with pytest.raises(CyclicDependencyError) as e:
        g.compile()
    assert isinstance(e.value, TaskGraphError) and "a" in str(e.value)


def test_batch_zero_input():
    g = G()
    t = g.linear(torch.randn(0, 256), torch.randn(512, 256))
    g.compile(); g.execute()
    assert t.output.shape == (0, 512)


def test_device_rule_cpu_graph_rejects_meta_and_accepts_cpu():
    g = G()
    g.linear(torch.randn(2, 4), torch.randn(4, 4))
    with pytest.raises(DeviceError) as e:
        g.linear(torch.empty(2, 4, device="meta"), torch.empty(4, 4, device="meta"))
    assert "meta" in str(e.value)


@pytest.mark.gpu
def test_cuda_graph_rejects_cpu_tensors():
    g = TaskGraph(num_workers=4)
    assert g.device.type == "cuda"
    with pytest.raises(DeviceError) as e:
        g.linear(torch.randn(2, 4), torch.randn(4, 4, device="cuda"))
    assert "cpu" in str(e.value)


def test_bad_reduce_op_and_unknown_activation():
    g = G()
    with pytest.raises(ValidationError):
        g.allreduce(torch.randn(4), op="xor")
    with pytest.raises(ValidationError):
        g.linear(torch.randn(2, 4), torch.randn(4, 4), activation="tanh")
