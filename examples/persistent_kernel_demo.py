#!/usr/bin/env python
"""The reference's two demo tables on this GPU (README.md:123-128 of the reference):

1. throughput of the barrier demo kernel with 1 / 2 / 4 / 8 ... worker CTAs over 1 Mi fp32 x 10 rounds;
2. 40 small tasks in ONE launch of the persistent kernel against 40 separate PyTorch launches.

    python examples/persistent_kernel_demo.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import maco_b200 as maco
from maco_b200.core import run_sm_scheduling_demo


def main():
    print("workers  ms      GB/s    scaling")
    base = None
    for ctas in (1, 2, 4, 8, 32, 148):
        data = torch.ones(1 << 20, device="cuda")
        run_sm_scheduling_demo(data, num_ctas=ctas, num_tasks=10)          # warm-up
        data.fill_(1.0)
        r = run_sm_scheduling_demo(data, num_ctas=ctas, num_tasks=10)
        base = base or r["gbs"]
        print(f"{ctas:7d}  {r['ms']:.4f}  {r['gbs']:7.1f}  {r['gbs'] / base:5.2f}x")

    # 40 dependent element-wise tasks on 1024 floats: one persistent launch vs 40 launches
    x = torch.randn(1024, device="cuda", dtype=torch.bfloat16)
    g = maco.TaskGraph()
    cur = x
    for i in range(40):
        cur = g.scale(cur, 1.01).output
    g.compile(runtime="persistent")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(iters):
            fn()
        ev1.record()
        torch.cuda.synchronize()
        return ev0.elapsed_time(ev1) / iters

    def eager():
        y = x
        for _ in range(40):
            y = y * 1.01
        return y

    t_one, t_many = timed(g.execute), timed(eager)
    print(f"40 tasks, one persistent launch: {t_one:.4f} ms; 40 separate launches: {t_many:.4f} ms; "
          f"ratio {t_many / t_one:.1f}x")


if __name__ == "__main__":
    main()
