"""Runs a function as N ranks in spawned processes (gloo on CPU, NCCL on GPUs)."""
import os
import socket
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errq, env):
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    os.environ.update(env)
    try:
        fn(rank, world, *args)
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world: int, args=(), timeout: float = 120.0, env=None, expect_fail_ranks=()):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq, dict(env or {}))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    hung = [i for i, p in enumerate(procs) if p.is_alive()]
    for i in hung:
        procs[i].kill()          # exact child processes started above
        procs[i].join()
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    bad = [(i, p.exitcode) for i, p in enumerate(procs) if p.exitcode != 0 and i not in expect_fail_ranks]
    assert not hung, f"ranks {hung} did not finish within {timeout}s"
    assert not bad, f"ranks failed: {bad}\n" + "\n".join(f"[rank {r}]\n{tb}" for r, tb in errors)
