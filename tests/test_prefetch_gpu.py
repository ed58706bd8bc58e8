"""InputPrefetcher: inputs arrive in submission order, staging buffers are reused safely."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_prefetcher_delivers_in_order():
    from maco_b200.utils import InputPrefetcher
    dst = torch.empty(1 << 20, device="cuda", dtype=torch.float32)
    feed = InputPrefetcher(dst)
    hosts = [torch.full((1 << 20,), float(i)).pin_memory() for i in range(5)]
    feed.submit(hosts[0])
    for i in range(5):
        feed.deliver(dst)
        if i + 1 < 5:
            feed.submit(hosts[i + 1])
        torch.cuda.current_stream().synchronize()
        assert torch.all(dst == i)
    assert feed.pending == 0
    with pytest.raises(RuntimeError):
        feed.deliver(dst)


def test_step_pipeline_results_lag_one_step():
    from maco_b200.utils import StepPipeline
    inp = torch.zeros(64, 32, device="cuda")
    out = torch.zeros(2, device="cuda")
    pipe = StepPipeline(inp, out)
    hosts = [torch.full((64, 32), float(i)).pin_memory() for i in range(5)]
    got = []
    for i in range(5):
        nxt = hosts[i + 1] if i + 1 < 5 else None
        r = pipe.step(hosts[i], lambda: out.copy_(inp[0, :2] * 2), lambda: out, next_host_input=nxt)
        got.append(None if r is None else r.clone())
    last = pipe.drain()
    assert got[0] is None
    for i in range(1, 5):
        assert torch.all(got[i] == 2.0 * (i - 1)), (i, got[i])
    assert torch.all(last == 8.0)


def test_step_pipeline_direct_delivery_into_two_slots():
    """Two input slots: every step sees ITS input (copied straight into the slot the previous launch does not
    read), results lag one step, buffers are never overwritten while a launch reads them."""
    from maco_b200.utils import StepPipeline
    slots = [torch.zeros(1 << 20, device="cuda"), torch.zeros(1 << 20, device="cuda")]
    out = torch.zeros(2, device="cuda")
    pipe = StepPipeline(slots, out)
    hosts = [torch.full((1 << 20,), float(i)).pin_memory() for i in range(7)]
    got = []
    for i in range(7):
        nxt = hosts[i + 1] if i + 1 < 7 else None
        r = pipe.step(hosts[i], lambda s: out.copy_(torch.stack([slots[s].min(), slots[s].max()])), lambda s: out,
                      next_host_input=nxt)
        got.append(None if r is None else r.clone())
    last = pipe.drain()
    assert got[0] is None
    for i in range(1, 7):
        assert torch.all(got[i] == float(i - 1)), (i, got[i])
    assert torch.all(last == 6.0)
