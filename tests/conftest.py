"""Shared fixtures. Tests that need a GPU carry ``@pytest.mark.gpu``; everything else runs on CPU
(multi-rank paths use the gloo backend with spawned processes)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least 2 CUDA devices")
    config.addinivalue_line("markers", "slow: long-running")


def pytest_collection_modifyitems(config, items):
    have_gpu = torch.cuda.is_available()
    ngpu = torch.cuda.device_count() if have_gpu else 0
    for item in items:
        if "gpu" in item.keywords and not have_gpu:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and ngpu < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)
    yield


@pytest.fixture
def device():
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


@pytest.fixture
def cpu_graph():
    import maco_b200 as maco
    return maco.TaskGraph(num_workers=4, device="cpu")


def assert_close(actual, expected, dtype=None):
    dtype = dtype or actual.dtype
    tol = {torch.float32: (1e-4, 1e-4), torch.float16: (1e-2, 1e-2), torch.bfloat16: (1e-1, 5e-2)}[dtype]
    torch.testing.assert_close(actual.float(), expected.float(), atol=tol[0], rtol=tol[1])
