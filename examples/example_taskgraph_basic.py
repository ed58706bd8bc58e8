#!/usr/bin/env python
"""Build, compile and run a small task graph (counterpart of the reference's
examples/example_taskgraph_basic.py). Runs on a GPU when there is one, else on the CPU."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import maco_b200 as maco


def main():
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    dt = torch.bfloat16 if dev == "cuda" else torch.float32
    x = torch.randn(256, 512, device=dev, dtype=dt)
    w1 = torch.randn(1024, 512, device=dev, dtype=dt) * 0.04
    w2 = torch.randn(512, 1024, device=dev, dtype=dt) * 0.03
    g = maco.TaskGraph(device=dev)
    t1 = g.linear(x, w1, activation="gelu", name="fc1")
    t2 = g.linear(t1.output, w2, name="fc2")
    t3 = g.add(t2.output, x, name="residual")
    g.compile()
    g.execute()
    if dev == "cuda":
        torch.cuda.synchronize()
    ref = torch.nn.functional.gelu(x.float() @ w1.float().t(), approximate="tanh") @ w2.float().t() + x.float()
    print(g.summary())
    print("max abs error vs fp32:", (t3.output.float() - ref).abs().max().item())


if __name__ == "__main__":
    main()
