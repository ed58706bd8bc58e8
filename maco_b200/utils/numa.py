"""Host-side placement for the end-to-end path: run this process on the CPUs next to its GPU.

A step that feeds its input from pinned host memory is bound by where that memory lives: on a two-socket host the
pages of a pinned buffer land on the socket of the thread that allocates them, and a GPU attached to the other
socket then pulls every input byte across the socket interconnect. With eight ranks started without placement the
aggregate host-to-device rate measured on an 8 x B200 host stayed near 100 GB/s (12 GB/s per GPU) whatever the number
of GPUs, which made the end-to-end step of the 4- and 8-GPU runs a copy-bound 675-705 us.

``bind_host_to_gpu`` restricts the calling process to the CPUs NVML reports as local to the GPU (intersected with
the CPUs the process may already use: a container's cpuset is respected, and an empty intersection leaves everything
unchanged). Call it before allocating pinned memory. It changes nothing on the GPU; it only calls
``os.sched_setaffinity`` for this process. The reference leaves placement to the launcher.
"""
from __future__ import annotations

import os
from typing import Dict


def _cuda_bus_id(device_index: int) -> str:
    import torch
    p = torch.cuda.get_device_properties(device_index)
    return "%08x:%02x:%02x.0" % (getattr(p, "pci_domain_id", 0), p.pci_bus_id, p.pci_device_id)


def local_cpus(device_index: int) -> set:
    """CPUs NVML reports as local to CUDA device ``device_index`` (empty set when unknown)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            try:
                h = pynvml.nvmlDeviceGetHandleByPciBusId(_cuda_bus_id(device_index).encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            words = (max(1, os.cpu_count() or 1) + 63) // 64
            mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
            cpus = set()
            for w, bits in enumerate(mask):
                bits = int(bits)
                for b in range(64):
                    if bits >> b & 1:
                        cpus.add(w * 64 + b)
            return cpus
        finally:
            pynvml.nvmlShutdown()
    except Exception:
        return set()


def bind_host_to_gpu(device_index: int) -> Dict[str, object]:
    """Restricts this process to the CPUs local to the GPU. Returns what happened:
    ``{"bound": bool, "cpus": n, "reason": str}``. ``MACO_NUMA_BIND=0`` turns it off."""
    if os.environ.get("MACO_NUMA_BIND", "1") == "0":
        return {"bound": False, "cpus": 0, "reason": "disabled by MACO_NUMA_BIND=0"}
    if not hasattr(os, "sched_setaffinity"):
        return {"bound": False, "cpus": 0, "reason": "no sched_setaffinity on this platform"}
    try:
        allowed = set(os.sched_getaffinity(0))
        near = local_cpus(device_index)
        if not near:
            return {"bound": False, "cpus": len(allowed), "reason": "NVML reports no CPU affinity for the device"}
        target = allowed & near
        if not target:
            return {"bound": False, "cpus": len(allowed), "reason": "none of the GPU-local CPUs is available to this process"}
        if target == allowed:
            return {"bound": False, "cpus": len(allowed), "reason": "already on GPU-local CPUs only"}
        os.sched_setaffinity(0, target)
        return {"bound": True, "cpus": len(target), "reason": "restricted to the GPU-local CPUs"}
    except Exception as e:                                        # placement is an optimisation, never a failure
        return {"bound": False, "cpus": 0, "reason": f"{type(e).__name__}: {e}"}
