"""Python entry point of the barrier self-test kernel (the reference's ``maco._sm.run_sm_scheduling_demo``,
maco/csrc/maco_kernel.cu:213-249): ``num_ctas`` co-resident CTAs run ``num_tasks`` rounds of
``x = x * 1.5 + 0.1`` over their slice of ``data`` with a bounded grid barrier between rounds."""
from __future__ import annotations

import ctypes
from typing import Dict

import torch

from .. import _native


def run_sm_scheduling_demo(data: torch.Tensor, num_ctas: int = 8, threads: int = 128, num_tasks: int = 10) -> Dict:
    """Runs the demo in place on fp32 ``data``; returns device time, effective bandwidth and the order in
    which the CTAs arrived at every barrier round."""
    if data.dtype != torch.float32 or not data.is_cuda or not data.is_contiguous():
        raise ValueError("run_sm_scheduling_demo needs a contiguous fp32 CUDA tensor")
    lib = _native.lib()
    lib.maco_run_sm_scheduling_demo.restype = ctypes.c_float
    lib.maco_run_sm_scheduling_demo.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                ctypes.c_void_p, ctypes.c_void_p]
    order = torch.zeros(num_ctas * num_tasks, dtype=torch.int32, device=data.device)
    ms = lib.maco_run_sm_scheduling_demo(data.data_ptr(), data.numel(), num_ctas, threads, num_tasks, order.data_ptr(),
                                         _native.current_stream_ptr())
    if ms < 0:
        raise RuntimeError(f"run_sm_scheduling_demo failed: {_native.last_error()}")
    nbytes = data.numel() * 4 * 2 * num_tasks                  # every round reads and writes the array
    return {"ms": float(ms), "gbs": nbytes / (ms * 1e-3) / 1e9, "order": order.view(num_tasks, num_ctas).cpu()}
