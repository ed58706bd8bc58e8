"""CPU model of the persistent kernel's scheduling protocol (csrc/host_sim/host_sim.cpp).

Builds ``libmaco_host_sim.so`` with g++ on first use (``MACO_HOST_SIM_TSAN=1`` adds
``-fsanitize=thread``) and runs task programs with threads standing in for CTAs: dependency
resolution, ring back-pressure, epochs, and injected faults, without a GPU.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path
from typing import List, Optional, Sequence, Tuple

import numpy as np

_SRC = Path(__file__).resolve().parents[2] / "csrc" / "host_sim" / "host_sim.cpp"
_LIB = Path(__file__).resolve().parents[1] / "_lib" / "libmaco_host_sim.so"

TASK = np.dtype([("wait_event", "<i4", 2), ("wait_count", "<u4", 2), ("signal_event", "<i4", 2), ("work_us", "<u4"),
                 ("stall", "<u4")])
GROUP = np.dtype([("first_task", "<u4"), ("num_tasks", "<u4"), ("wait_event", "<i4", 2), ("wait_count", "<u4", 2)])
STATUS_TIMEOUT, STATUS_BAD_TASK, STATUS_QUEUE_OVERFLOW = 1, 2, 4

_lib = None


def build(force: bool = False) -> Path:
    if _LIB.exists() and not force and _LIB.stat().st_mtime >= _SRC.stat().st_mtime:
        return _LIB
    _LIB.parent.mkdir(parents=True, exist_ok=True)
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", str(_SRC), "-o", str(_LIB)]
    if os.environ.get("MACO_HOST_SIM_TSAN") == "1":
        cmd[1:1] = ["-fsanitize=thread", "-g"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{res.stderr}")
    return _LIB


def _load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(build()))
        a, b = ctypes.c_int(), ctypes.c_int()
        lib.maco_host_sim_sizes(ctypes.byref(a), ctypes.byref(b))
        assert (a.value, b.value) == (TASK.itemsize, GROUP.itemsize), "host_sim ABI mismatch"
        _lib = lib
    return _lib


def groups_of(tasks: np.ndarray) -> np.ndarray:
    """Dispatch groups = maximal runs of consecutive tasks with identical wait conditions."""
    out, i, n = [], 0, len(tasks)
    key = lambda t: (tuple(t["wait_event"]), tuple(t["wait_count"]))
    while i < n:
        j = i + 1
        while j < n and key(tasks[j]) == key(tasks[i]):
            j += 1
        out.append((i, j - i, tuple(tasks[i]["wait_event"]), tuple(tasks[i]["wait_count"])))
        i = j
    g = np.zeros(len(out), dtype=GROUP)
    for k, (f, c, we, wc) in enumerate(out):
        g[k]["first_task"], g[k]["num_tasks"], g[k]["wait_event"], g[k]["wait_count"] = f, c, we, wc
    return g


def run(tasks: np.ndarray, num_events: int, num_workers: int, mode: str = "static", ring_size: int = 1024,
        epochs: int = 1, budget_ms: float = 2000.0) -> dict:
    """Runs the program; returns status bits, failing task / event, completed count and completion order."""
    lib = _load()
    tasks = np.ascontiguousarray(tasks, dtype=TASK)
    groups = groups_of(tasks)
    queues: List[List[int]] = [[] for _ in range(num_workers)]
    for i in range(len(tasks)):
        queues[i % num_workers].append(i)
    stride = max(1, max(len(q) for q in queues))
    sq = np.full((num_workers, stride), 0xFFFFFFFF, dtype=np.uint32)
    for w, q in enumerate(queues):
        sq[w, : len(q)] = q
    sc = np.array([len(q) for q in queues], dtype=np.uint32)
    order = np.full(max(1, len(tasks) * epochs), 0xFFFFFFFF, dtype=np.uint32)
    result = np.zeros(4, dtype=np.uint32)
    P = ctypes.c_void_p
    rc = lib.maco_host_sim_run(P(tasks.ctypes.data), len(tasks), P(groups.ctypes.data), len(groups), num_events, num_workers,
                               ring_size, 1 if mode == "dynamic" else 0, P(sq.ctypes.data), P(sc.ctypes.data), stride,
                               epochs, ctypes.c_uint64(int(budget_ms * 1000)), P(order.ctypes.data), P(result.ctypes.data))
    if rc != 0:
        raise RuntimeError("maco_host_sim_run rejected its arguments")
    done = int(result[3])
    return {"status": int(result[0]), "fail_task": int(result[1]), "fail_event": int(result[2]), "completed": done,
            "order": order[:done].tolist()}
