#!/usr/bin/env python
"""Plan a multi-GPU layer on a machine without GPUs: build every rank's program, check that the static
schedules cannot deadlock, and estimate the length of the launch.

    python examples/plan_schedule.py --world 8 --comm-workers 16

Builds the tensor-parallel SwiGLU MLP (8192 tokens, 4096 -> 14336) for every rank of a ``--world``-rank job on CPU
tensors over ``PlanningHeap`` stand-ins, runs the queues with ``simulate_static_queues`` (the kernel's rules: queue
order, two wait conditions per task, two-CTA halves together, peer signals) and prints what ``estimate_makespan``
predicts for a few choices of communication workers. The reference has no counterpart: its scheduler's plans are
only ever executed.
"""
import argparse
import os
import struct
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from maco_b200.models.tp_mlp import TPSwiGLUMLP
from maco_b200.ops import megakernel as mk
from maco_b200.parallel.symm_heap import PlanningHeap


def programs(world, comm_workers, tokens, hidden, ffn):
    out = []
    for rank in range(world):
        layer = TPSwiGLUMLP(tokens, hidden, ffn, rank=rank, world=world, heap=PlanningHeap(rank, world) if world > 1 else None,
                            device=torch.device("cpu"), comm_workers=comm_workers)
        b = layer.builders[0]
        out.append((b.tasks, mk.assign_static_queues(b.tasks, b.num_workers, b.num_comm_workers)))
    return out


def cost(task):
    """GEMM k-blocks at the rate measured for 256 x 256 two-CTA tiles on B200 (24.5 us for K = 4096); the rest as built in."""
    if task["type"] in (100, 101, 102):
        return 1.5 + 0.36 * struct.unpack_from("<i", task["raw"], 20)[0]
    return mk.default_task_cost(task)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--comm-workers", type=int, nargs="*", default=[8, 12, 16, 24])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    args = ap.parse_args()
    for cw in args.comm_workers:
        progs = programs(args.world, cw, args.tokens, args.hidden, args.ffn)
        rounds = mk.simulate_static_queues(progs)
        est = mk.estimate_makespan(progs, cost=cost)
        ends = est["last_end_by_type_us"][0]
        print(f"world {args.world}, {cw:2d} communication workers: {len(progs[0][0])} tasks per rank, schedule completes "
              f"({rounds} rounds); predicted launch {est['span_us'][0]:.0f} us, tiles end {ends.get(101, 0):.0f} us, "
              f"all-gather ends {ends.get(201, 0):.0f} us, workers busy {100 * est['busy_fraction'][0]:.0f} %")


if __name__ == "__main__":
    main()
