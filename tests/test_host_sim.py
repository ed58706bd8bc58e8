"""Scheduling protocol of the persistent kernel on the CPU model: dependencies, back-pressure, epochs,
and failure detection with host-side fault injection (a stalled worker, a missing producer)."""
import numpy as np
import pytest

from maco_b200.utils import host_sim as hs


def _chain_program(width=6, depth=5, work_us=0):
    """depth layers of `width` tasks; every task of layer l waits for ALL tasks of layer l-1."""
    tasks = np.zeros(width * depth, dtype=hs.TASK)
    tasks["wait_event"] = -1
    tasks["signal_event"] = -1
    for l in range(depth):
        for i in range(width):
            t = tasks[l * width + i]
            t["signal_event"][0] = l
            t["work_us"] = work_us
            if l > 0:
                t["wait_event"][0], t["wait_count"][0] = l - 1, width
    return tasks, depth


@pytest.mark.parametrize("mode", ["static", "dynamic"])
@pytest.mark.parametrize("workers", [1, 3, 8])
def test_dependencies_hold_and_epochs_repeat(mode, workers):
    tasks, ne = _chain_program()
    res = hs.run(tasks, ne, workers, mode=mode, epochs=3)
    assert res["status"] == 0 and res["completed"] == 3 * len(tasks)
    width = 6
    for ep in range(3):
        order = res["order"][ep * len(tasks):(ep + 1) * len(tasks)]
        pos = {t: i for i, t in enumerate(order)}
        assert sorted(order) == list(range(len(tasks)))
        for t in range(width, len(tasks)):          # every producer of the previous layer finished first
            assert all(pos[p] < pos[t] for p in range((t // width - 1) * width, (t // width) * width))


def test_ring_backpressure_with_tiny_rings():
    tasks, ne = _chain_program(width=16, depth=8, work_us=20)
    res = hs.run(tasks, ne, num_workers=2, mode="dynamic", ring_size=2, epochs=2)
    assert res["status"] == 0 and res["completed"] == 2 * len(tasks)


@pytest.mark.parametrize("mode", ["static", "dynamic"])
def test_missing_producer_times_out_and_reports_the_event(mode):
    tasks, ne = _chain_program(width=4, depth=3)
    tasks[5]["wait_event"][1], tasks[5]["wait_count"][1] = ne, 1      # an event nothing signals
    res = hs.run(tasks, ne + 1, 4, mode=mode, budget_ms=50)
    assert res["status"] & hs.STATUS_TIMEOUT
    assert res["completed"] < len(tasks)
    if mode == "static":
        # the first waiter whose budget runs out reports: task 5 itself, or (threads are scheduled by the host,
        # budgets start within microseconds of each other) a task of the next layer that waits for task 5's layer
        assert (res["fail_task"], res["fail_event"]) == (5, ne) or res["fail_task"] >= 8


@pytest.mark.parametrize("mode", ["static", "dynamic"])
def test_stalled_worker_is_detected_by_its_consumers(mode):
    tasks, ne = _chain_program(width=4, depth=3)
    tasks[2]["stall"] = 1                        # injected on the host: this task never finishes
    res = hs.run(tasks, ne, 4, mode=mode, budget_ms=50)
    assert res["status"] & hs.STATUS_TIMEOUT
    assert 2 not in res["order"] and res["completed"] < len(tasks)
