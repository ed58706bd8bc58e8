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
