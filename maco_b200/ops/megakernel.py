"""Host side of the persistent task kernel: program builder, graph lowering, launch.

``ProgramBuilder`` turns operations into tile-granular task descriptors with (event, count) wait
conditions and signals; ``Program`` owns the device tables and launches ``maco_persistent_kernel``
once per ``run()``; ``lower_graph`` maps a compiled ``TaskGraph`` onto a builder.

The reference's ``MacoRuntime`` (maco/task_graph/runtime.py:21-144) re-uploads every task on every
execute with three host syncs each and forwards only the first input and first dependency. Here
the whole table is built at compile time, uploaded in one copy, and ``run()`` is: bump the epoch,
one launch.
"""
from __future__ import annotations

import collections
import ctypes
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native as N
from ..task_graph.nodes import TaskNode, TaskType

BM, BK = 128, 64
QUEUE_TERMINATE = 0xFFFFFFFF
MODE_STATIC, MODE_DYNAMIC = 0, 1
TF_WAIT0_SYS, TF_WAIT1_SYS, TF_COMM_WORKER, TF_SIGNAL_SYS, TF_WAIT0_PREV, TF_WAIT1_PREV = 1, 2, 4, 8, 16, 32
TF_ANY_WORKER = 64      # host-side placement hint: spread over compute AND communication workers
TF_COUNTED = 128        # GEMM tile guarded by a run-time row count
COMM_PUSH, COMM_REDUCE_LOCAL, COMM_REDUCE_PULL, COMM_ALLREDUCE, COMM_ALLREDUCE_MC, COMM_PULL, COMM_REDUCE_LOCAL_BCAST, COMM_PUSH_MC = range(8)
MAX_PEERS = 16
WORKER_QUEUE_SIZE = 1024
T_SPLITK_FIN = 118

EPI = {None: 0, "none": 0, "gelu": 1, "swiglu": 2, "f32": 3, "f32_acc": 4, "gelu_bwd": 5, "silu": 6, "residual": 7, "f32_atomic": 8,
       "splitk_fused": 9, "scatter_rows": 10}

TASK_DTYPE = np.dtype([
    ("type", "<u2"), ("flags", "<u2"), ("node_id", "<u4"), ("wait_event", "<i4", 2), ("wait_count", "<u4", 2),
    ("signal_event", "<i4", 2), ("signal_peer", "<i4"), ("signal_peer_event", "<i4"), ("raw", "u1", 88),
])
GROUP_DTYPE = np.dtype([
    ("first_task", "<u4"), ("num_tasks", "<u4"), ("wait_event", "<i4", 2), ("wait_count", "<u4", 2),
    ("flags", "<u4"), ("_pad", "<u4"),
])
TRACE_DTYPE = np.dtype([("task", "<u4"), ("type", "<u2"), ("sm", "<u2"), ("t_start_ns", "<u8"), ("t_end_ns", "<u8"),
                        ("wait_ns", "<u8")])


class _ProgramStruct(ctypes.Structure):
    _fields_ = [
        ("tasks", ctypes.c_void_p), ("tmaps", ctypes.c_void_p), ("epis", ctypes.c_void_p), ("events", ctypes.c_void_p),
        ("peer_events", ctypes.c_void_p * MAX_PEERS), ("peer_heap", ctypes.c_void_p * MAX_PEERS),
        ("static_queue", ctypes.c_void_p), ("static_count", ctypes.c_void_p), ("ring", ctypes.c_void_p),
        ("heads", ctypes.c_void_p), ("tails", ctypes.c_void_p), ("groups", ctypes.c_void_p),
        ("abort_word", ctypes.c_void_p), ("counters", ctypes.c_void_p), ("mc_heap", ctypes.c_void_p),
        ("status", ctypes.c_void_p), ("trace", ctypes.c_void_p), ("budget_ns", ctypes.c_ulonglong),
        ("num_tasks", ctypes.c_uint32), ("num_groups", ctypes.c_uint32), ("num_workers", ctypes.c_uint32),
        ("num_comm_workers", ctypes.c_uint32), ("static_stride", ctypes.c_uint32), ("mode", ctypes.c_uint32),
        ("epoch", ctypes.c_uint32), ("rank", ctypes.c_int32), ("world", ctypes.c_int32),
        ("cta_group", ctypes.c_uint32), ("debug", ctypes.c_uint32), ("heap_bytes", ctypes.c_uint64),
        ("num_events", ctypes.c_uint32), ("num_tmaps", ctypes.c_uint32), ("num_epis", ctypes.c_uint32), ("_pad", ctypes.c_uint32),
    ]


_abi_checked = False


def _lib():
    global _abi_checked
    lib = N.lib()
    if not _abi_checked:
        I, P, LL = ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong
        lib.maco_abi_sizes.restype = I
        lib.maco_abi_sizes.argtypes = [ctypes.POINTER(I)] * 6
        lib.maco_encode_operand_tmap.restype = I
        lib.maco_encode_operand_tmap.argtypes = [P, P, I, I, LL, I, I]
        lib.maco_program_launch.restype = I
        lib.maco_program_launch.argtypes = [ctypes.POINTER(_ProgramStruct), P]
        lib.maco_persistent_smem_bytes.restype = I
        lib.maco_persistent_max_pairs.restype = I
        sizes = [I() for _ in range(6)]
        lib.maco_abi_sizes(*[ctypes.byref(s) for s in sizes])
        got = [s.value for s in sizes]
        want = [TASK_DTYPE.itemsize, GROUP_DTYPE.itemsize, ctypes.sizeof(_ProgramStruct), 72, TRACE_DTYPE.itemsize, 128]
        if got != want:
            raise RuntimeError(f"ABI mismatch between the Python tables and libmaco_b200: native {got}, python {want}")
        _abi_checked = True
    return lib


def _pack_gemm(tmap_a, tmap_b, epi, a_mn, b_mn, m0, n0, k0, k_blocks, idesc, peer, row_off, out_off, bn, count_base=0,
               count_ptr=0) -> bytes:
    return struct.pack("<HHHBBiiiiIiqQIIQ", tmap_a, tmap_b, epi, a_mn, b_mn, m0, n0, k0, k_blocks, idesc, peer, row_off,
                       out_off, bn, count_base, count_ptr or 0)


def _pack_elt(in0, in1, in2, out, row0, rows, cols, dtype, ld_in, ld_out, f0=0.0, f1=0.0, i0=0, i1=0) -> bytes:
    return struct.pack("<QQQQiiiiiiffii", in0 or 0, in1 or 0, in2 or 0, out or 0, row0, rows, cols, dtype, ld_in, ld_out,
                       f0, f1, i0, i1)


def _pack_comm(src_off, dst_off, src_stride, dst_stride, row_bytes, rows, dtype, peer, op, nslots=0, slot_stride=0,
               local_ptr=0, scale=1.0, aux_ptr=0) -> bytes:
    return struct.pack("<QQQQIIiiiiQQfiQ", src_off, dst_off, src_stride, dst_stride, row_bytes, rows, dtype, peer, op,
                       nslots, slot_stride, local_ptr or 0, scale, 0, aux_ptr or 0)


def _pack_epilogue(out, bias, aux, ld_out, ld_aux, mode, out_type, bias_type, aux_type, M, Nn, alpha, aux_pack=0) -> bytes:
    return struct.pack("<QQQqqiiiiiifi", out or 0, bias or 0, aux or 0, ld_out, ld_aux, mode, out_type, bias_type,
                       aux_type, M, Nn, alpha, aux_pack)


def make_idesc(ab_format: int, m: int, n: int, a_mn: int, b_mn: int) -> int:
    return (1 << 4) | (ab_format << 7) | (ab_format << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24)


Wait = Tuple[int, int, int]   # (event, count, flags among SYS/PREV expressed for slot 0)


def pick_split_k(n_tiles: int, k_blocks: int, workers: int) -> int:
    """K slices of a few-row GEMM: minimises waves of tiles over the workers x (k-blocks per tile + a fixed
    cost per tile for pipeline fill and the reductions)."""
    def cost(sp: int) -> int:
        return -(-n_tiles * sp // workers) * (-(-k_blocks // sp) + 8)
    return min(range(1, max(1, min(16, k_blocks // 2)) + 1), key=cost)


def attention_pieces(groups: int, kv_len: int, workers: int) -> List[Tuple[int, int, int, int]]:
    """Cuts ``groups`` key ranges of ``kv_len`` keys into one (nearly) equal share per worker.
    Returns (group, first key, keys, worker); cuts inside a group sit on 128-key boundaries."""
    target = -(-(groups * kv_len) // workers)
    target = -(-target // 128) * 128
    pieces, wk, acc = [], 0, 0
    for g in range(groups):
        s0 = 0
        while s0 < kv_len:
            room = target - acc                     # > 0 here
            take = min(kv_len - s0, -(-room // 128) * 128)
            pieces.append((g, s0, take, min(wk, workers - 1)))
            s0 += take
            acc += take
            if acc >= target:
                wk, acc = wk + 1, 0
    return pieces



@dataclass
class RowEvents:
    """Completion events of a produced 2-D tensor: one per ``block`` rows plus one for the whole tensor."""
    rows: int
    block: int
    row_events: List[Tuple[int, int]]          # (event, count) per row block
    all_event: Tuple[int, int]                 # (event, count) of the whole node
    sys: bool = False                          # signalled by other GPUs

    def for_rows(self, r0: int, r1: int) -> Tuple[int, int]:
        b0, b1 = r0 // self.block, (max(r0 + 1, r1) - 1) // self.block
        if b0 == b1 and b0 < len(self.row_events):
            return self.row_events[b0]
        return self.all_event


def assign_static_queues(tasks: Sequence[dict], num_workers: int, num_comm_workers: int) -> List[List[int]]:
    """Static per-worker queues of a program: the tasks in emission (= a topological) order, round-robin over the
    worker class each task prefers. Pure host code (no device needed), so schedules can be checked on a CPU
    (``simulate_static_queues``)."""
    W, Wc = num_workers, num_comm_workers
    n_compute = W - Wc
    queues: List[List[int]] = [[] for _ in range(W)]
    rr_c = rr_m = rr_a = rr_p = 0
    n_pairs = max(1, n_compute // 2)
    pair_of_leader = 0
    attached: Dict[int, List[int]] = {}             # task -> join tasks that run right in front of it
    for i, t in enumerate(tasks):
        if t.get("attach_to") is not None:
            # Still a topological order: a join's only consumer is the task it is attached to.
            attached.setdefault(t["attach_to"], []).append(i)
            continue
        if t.get("pair_half") is not None:
            # halves of a two-CTA tile: consecutive tasks, leader on worker 2j, the other half on 2j+1; both
            # workers see their pair tiles in the same order (the MMA of one serves both)
            if t["pair_half"] == 0:
                pair_of_leader = (rr_p + rr_p // n_pairs) % n_pairs
                rr_p += 1
            q = 2 * pair_of_leader + t["pair_half"]
        elif (t["flags"] & TF_ANY_WORKER) and Wc > 0:
            q = (W - 1 - rr_a) % W                     # communication workers (highest indices) first
            rr_a += 1
        elif (t["flags"] & TF_COMM_WORKER) and Wc > 0:
            q = n_compute + rr_m % Wc
            rr_m += 1
        elif t.get("worker") is not None:
            q = t["worker"] % n_compute
        else:
            # rotate by one worker per wave: with a plain modulo a worker would see the same position of
            # every periodic task pattern (the same row block of every expert slab, say) and the load
            # would follow that pattern instead of averaging out
            q = (rr_c + rr_c // n_compute) % n_compute
            rr_c += 1
        queues[q] += attached.pop(i, [])
        queues[q].append(i)
    if attached:
        raise RuntimeError("join tasks attached to a task that was never emitted")
    return queues


def simulate_static_queues(programs: Sequence[Tuple[Sequence[dict], List[List[int]]]], max_rounds: int = 1 << 22) -> int:
    """Runs the static schedules of one program per rank on the host, with the rules of the kernel: a worker runs the
    head of its queue once both wait conditions hold (event counter >= count; "previous launch" conditions hold at
    once in a first launch), the two halves of a two-CTA tile only run together, a finished task bumps its local
    events and the events it signals on a peer (-2 / -4: on every rank). Returns the number of rounds; raises
    RuntimeError with the stuck queue heads if no task can run (a deadlock of the schedule). Counted (run-time
    skipped) tiles and time are not modelled: this checks the ORDER of the queues, on any machine."""
    world = len(programs)
    events = [collections.defaultdict(int) for _ in range(world)]
    heads = [[0] * len(q) for _, q in programs]
    left = sum(len(t) for t, _ in programs)

    def ready(r: int, t: dict) -> bool:
        for k in range(2):
            ev, cnt = t["wait_event"][k], t["wait_count"][k]
            prev = t["flags"] & (TF_WAIT0_PREV if k == 0 else TF_WAIT1_PREV)
            if ev >= 0 and cnt > 0 and not prev and events[r][ev] < cnt:
                return False
        return True

    def finish(r: int, t: dict) -> None:
        for ev in t["signal_event"]:
            if ev >= 0:
                events[r][ev] += 1
        sp, spe = t["signal_peer"], t["signal_peer_event"]
        if spe >= 0 and sp != -1:
            for d in (range(world) if sp in (-2, -4) else [sp]):
                events[d][spe] += 1

    rounds = 0
    while left:
        rounds += 1
        if rounds > max_rounds:
            raise RuntimeError("simulate_static_queues: round limit reached")
        progressed = False
        for r, (tasks, queues) in enumerate(programs):
            for w, q in enumerate(queues):
                h = heads[r][w]
                if h >= len(q):
                    continue
                t = tasks[q[h]]
                if not ready(r, t):
                    continue
                half = t.get("pair_half")
                if half is None:
                    finish(r, t)
                    heads[r][w] += 1
                    left -= 1
                    progressed = True
                elif half == 0:
                    # leader half: its partner (worker w + 1) must be at the other half of the same tile, ready
                    hp = heads[r][w + 1]
                    qp = queues[w + 1]
                    if hp < len(qp) and qp[hp] == q[h] + 1 and ready(r, tasks[qp[hp]]):
                        finish(r, t)
                        finish(r, tasks[qp[hp]])
                        heads[r][w] += 1
                        heads[r][w + 1] += 1
                        left -= 2
                        progressed = True
                # half == 1 runs with its leader
        if not progressed:
            stuck = []
            for r, (tasks, queues) in enumerate(programs):
                for w, q in enumerate(queues):
                    if heads[r][w] < len(q):
                        t = tasks[q[heads[r][w]]]
                        stuck.append((r, w, q[heads[r][w]], t["type"], t["wait_event"], t["wait_count"],
                                      [events[r][e] for e in t["wait_event"] if e >= 0]))
            raise RuntimeError(f"static schedule deadlocks; stuck queue heads (rank, worker, task, type, waits, counts, "
                               f"values): {stuck[:8]}")
    return rounds


def default_task_cost(t: dict) -> float:
    """Rough duration of a task in microseconds for ``estimate_makespan``, from figures measured on B200 with this
    kernel: a 128 x 256 x 64 k-block of a GEMM tile 0.45 us (a pair half the same: two CTAs, twice the rows) plus 2 us
    per tile; a bulk push 43 us per MB; a staged reduction 0.06 us per KB of sources; everything else 5 us. Callers
    with better numbers for their shapes pass their own function."""
    ty = t["type"]
    raw = t["raw"]
    if ty in (100, 101, 102) and len(raw) >= 30:
        k_blocks = struct.unpack_from("<i", raw, 20)[0]
        return 2.0 + 0.45 * max(1, k_blocks)
    if 200 <= ty < 300 and len(raw) >= 40:
        row_bytes, rows = struct.unpack_from("<II", raw, 32)
        op = struct.unpack_from("<i", raw, 48)[0]
        nbytes = row_bytes * rows
        if op in (COMM_REDUCE_LOCAL, COMM_REDUCE_LOCAL_BCAST, COMM_ALLREDUCE):
            nslots = max(1, struct.unpack_from("<i", raw, 52)[0])
            return 4.0 + 0.06 * nbytes * nslots / 1024.0
        return 3.0 + 43.0 * nbytes / (1 << 20)
    return 5.0


def estimate_makespan(programs: Sequence[Tuple[Sequence[dict], List[List[int]]]], cost=default_task_cost,
                      hop_us: float = 2.0) -> Dict[str, object]:
    """Discrete-event run of the static schedules of one program per rank with task durations from ``cost(task)``
    (microseconds) and ``hop_us`` between a signal and the waiter seeing it. Same rules as ``simulate_static_queues``
    (queue order, both wait conditions, pair halves together, peer signals). Returns the predicted length of the launch
    per rank, the busy fraction of the workers and the last finish time per task type: a planning aid for choosing the
    number of communication workers, chunk sizes and tile orders before a GPU is involved, not a measurement."""
    import heapq
    world = len(programs)
    counts = [collections.defaultdict(int) for _ in range(world)]
    heads = [[0] * len(q) for _, q in programs]
    free_at = [[0.0] * len(q) for _, q in programs]
    running = [[False] * len(q) for _, q in programs]
    busy = [0.0] * world
    end_by_type = [collections.defaultdict(float) for _ in range(world)]
    left = sum(len(t) for t, _ in programs)
    pq: List[tuple] = []          # (time, seq, kind, rank, payload)
    seq = 0

    def ready(r: int, t: dict) -> bool:
        for k in range(2):
            ev, cnt = t["wait_event"][k], t["wait_count"][k]
            prev = t["flags"] & (TF_WAIT0_PREV if k == 0 else TF_WAIT1_PREV)
            if ev >= 0 and cnt > 0 and not prev and counts[r][ev] < cnt:
                return False
        return True

    def try_start(r: int, w: int, now: float) -> None:
        nonlocal seq
        tasks, queues = programs[r]
        q = queues[w]
        if running[r][w] or heads[r][w] >= len(q):
            return
        t = tasks[q[heads[r][w]]]
        half = t.get("pair_half")
        if half == 1:
            w = w - 1                                # the leader decides for the pair
            q = queues[w]
            if running[r][w] or heads[r][w] >= len(q):
                return
            t = tasks[q[heads[r][w]]]
            half = t.get("pair_half")
            if half != 0:
                return
        if not ready(r, t):
            return
        members = [(w, t)]
        if half == 0:
            qp = queues[w + 1]
            hp = heads[r][w + 1]
            if running[r][w + 1] or hp >= len(qp) or qp[hp] != q[heads[r][w]] + 1 or not ready(r, tasks[qp[hp]]):
                return
            members.append((w + 1, tasks[qp[hp]]))
        start = max([now] + [free_at[r][m] for m, _ in members])
        dur = max(cost(tt) for _, tt in members)
        for m, tt in members:
            running[r][m] = True
            busy[r] += dur
            seq += 1
            heapq.heappush(pq, (start + dur, seq, 0, r, (m, tt)))

    for r in range(world):
        for w in range(len(programs[r][1])):
            try_start(r, w, 0.0)
    now = 0.0
    while pq:
        now, _, kind, r, payload = heapq.heappop(pq)
        if kind == 0:                                # a task finishes on worker m of rank r
            m, t = payload
            running[r][m] = False
            free_at[r][m] = now
            heads[r][m] += 1
            left -= 1
            end_by_type[r][t["type"]] = max(end_by_type[r][t["type"]], now)
            for ev in t["signal_event"]:
                if ev >= 0:
                    seq += 1
                    heapq.heappush(pq, (now + hop_us, seq, 1, r, ev))
            sp, spe = t["signal_peer"], t["signal_peer_event"]
            if spe >= 0 and sp != -1:
                for d in (range(world) if sp in (-2, -4) else [sp]):
                    seq += 1
                    heapq.heappush(pq, (now + hop_us, seq, 1, d, spe))
            try_start(r, m, now)
            if t.get("pair_half") == 0:
                pass
        else:                                        # a signal becomes visible on rank r
            counts[r][payload] += 1
            for w in range(len(programs[r][1])):
                try_start(r, w, now)
    if left:
        raise RuntimeError("estimate_makespan: the schedule did not run to completion (see simulate_static_queues)")
    span = [max((free_at[r][w] for w in range(len(programs[r][1]))), default=0.0) for r in range(world)]
    return {"span_us": span,
            "busy_fraction": [busy[r] / max(1e-9, span[r] * len(programs[r][1])) for r in range(world)],
            "last_end_by_type_us": [dict(end_by_type[r]) for r in range(world)]}


class ProgramBuilder:
    """Accumulates tasks, events, tensor maps and epilogues; ``build()`` uploads them."""

    def __init__(self, device: torch.device, num_workers: Optional[int] = None, mode: str = "static",
                 num_comm_workers: int = 0, heap=None, trace: bool = False, wait_budget_ms: Optional[float] = None,
                 cta_pair: bool = False):
        """``cta_pair``: every GEMM tile of the program is computed by TWO CTAs (workers 2j and 2j+1, one
        thread-block cluster) with ``tcgen05.mma.cta_group::2``: 256 x bn per pair, each CTA loading its own 128
        rows of A and its own half of B. Static queues only; split-K, counted (MoE) and tensor-core attention
        tasks stay in one-CTA programs (a kernel has one cta_group)."""
        self.device = torch.device(device)
        # (a CPU device gives a planning-only builder: tasks and queues can be produced and checked, not built)
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 148
        self.mode = MODE_DYNAMIC if mode == "dynamic" else MODE_STATIC
        self.cta_pair = bool(cta_pair)
        if self.cta_pair and self.mode != MODE_STATIC:
            raise ValueError("two-CTA programs run with static queues")
        limit = sms - (1 if self.mode == MODE_DYNAMIC else 0)
        self.num_workers = max(1, min(int(num_workers) if num_workers else limit, limit, 256))
        self.num_comm_workers = max(0, min(int(num_comm_workers), self.num_workers - 1))
        if self.cta_pair:
            max_pairs = _lib().maco_persistent_max_pairs() if self.device.type == "cuda" else 0
            if max_pairs > 0:
                self.num_workers = min(self.num_workers, 2 * max_pairs)
            self.num_workers -= self.num_workers & 1
            self.num_comm_workers += self.num_comm_workers & 1          # compute workers come in pairs
            if self.num_workers < 2 or self.num_workers - self.num_comm_workers < 2:
                raise ValueError("two-CTA programs need at least one pair of compute workers")
        self.heap = heap
        self.trace = trace
        from ..config import config
        self.wait_budget_ms = float(wait_budget_ms if wait_budget_ms is not None else config.wait_budget_ms)
        self.tasks: List[dict] = []
        self.groups: List[dict] = []
        self.tmaps: List[bytes] = []
        self._tmap_cache: Dict[tuple, int] = {}
        self.epis: List[bytes] = []
        self.num_events = 0
        self.keepalive: List[torch.Tensor] = []
        self.launch_state: List[torch.Tensor] = []     # buffers that must be zero when the FIRST launch starts
        self._node_counter = 0

    # ------------------------------------------------------------------ primitives
    def new_event(self) -> int:
        e = self.num_events
        self.num_events += 1
        return e

    def new_node_id(self) -> int:
        self._node_counter += 1
        return self._node_counter - 1

    def add_task(self, ttype: int, raw: bytes, waits: Sequence[Tuple[int, int, bool, bool]] = (),
                 signals: Sequence[int] = (), signal_peer: int = -1, signal_peer_event: int = -1, node_id: int = 0,
                 comm_worker: bool = False, signal_sys: bool = False, any_worker: bool = False,
                 counted: bool = False, worker: Optional[int] = None, pair_half: Optional[int] = None) -> int:
        """``waits``: up to two (event, count, sys_scope, previous_epoch). ``worker`` pins the task to a compute
        worker's static queue (the dynamic scheduler ignores it)."""
        if len(waits) > 2 or len(signals) > 2:
            raise ValueError("a task takes at most two wait conditions and two local signals")
        flags = 0
        we, wc = [-1, -1], [0, 0]
        for j, (ev, cnt, sys_scope, prev) in enumerate(waits):
            we[j], wc[j] = ev, cnt
            if sys_scope:
                flags |= TF_WAIT0_SYS if j == 0 else TF_WAIT1_SYS
            if prev:
                flags |= TF_WAIT0_PREV if j == 0 else TF_WAIT1_PREV
        if comm_worker:
            flags |= TF_COMM_WORKER
        if signal_sys:
            flags |= TF_SIGNAL_SYS
        if any_worker:
            flags |= TF_ANY_WORKER
        if counted:
            flags |= TF_COUNTED
        se = list(signals) + [-1] * (2 - len(signals))
        self.tasks.append(dict(type=ttype, flags=flags, node_id=node_id, wait_event=we, wait_count=wc, signal_event=se,
                               signal_peer=signal_peer, signal_peer_event=signal_peer_event, raw=raw, worker=worker,
                               pair_half=pair_half))
        return len(self.tasks) - 1

    def join(self, waits: List[Tuple[int, int, bool, bool]], node_id: int = 0) -> List[Tuple[int, int, bool, bool]]:
        """Reduces a list of wait conditions to at most two with a balanced tree of NOP tasks (depth log2 n: a
        chain of n would add one dependency hop of a few microseconds per condition)."""
        waits = list(dict.fromkeys(waits))
        while len(waits) > 2:
            nxt = []
            for i in range(0, len(waits) - 1, 2):
                ev = self.new_event()
                self.add_task(int(TaskType.NOP), b"", waits=waits[i:i + 2], signals=[ev], node_id=node_id)
                nxt.append((ev, 1, False, False))
            if len(waits) % 2:
                nxt.append(waits[-1])
            waits = nxt
        return waits

    def _tmap(self, t: torch.Tensor, rows: int, cols: int, ld: int, mn_major: bool, box_rows: int) -> int:
        key = (t.data_ptr(), rows, cols, ld, mn_major, box_rows)
        idx = self._tmap_cache.get(key)
        if idx is not None:
            return idx
        if self.device.type != "cuda":
            # planning mode: tensor maps are encoded by the CUDA driver; the task lists do not need their contents
            self.tmaps.append(b"\0" * 128)
            self._tmap_cache[key] = len(self.tmaps) - 1
            return len(self.tmaps) - 1
        buf = ctypes.create_string_buffer(128)
        rc = _lib().maco_encode_operand_tmap(buf, t.data_ptr(), rows, cols, ld, int(mn_major), box_rows)
        N.check(rc, "maco_encode_operand_tmap")
        self.tmaps.append(buf.raw)
        self._tmap_cache[key] = len(self.tmaps) - 1
        return len(self.tmaps) - 1

    # ------------------------------------------------------------------ GEMM node
    def add_epilogue(self, out_ptr: int, ld_out: int, out_dtype: torch.dtype, M: int, Nn: int, *, mode: str = None,
                     aux_ptr: int = 0, ld_aux: int = 0, aux_dtype: Optional[torch.dtype] = None, alpha: float = 1.0,
                     aux_slots: Optional[Tuple[int, int, int]] = None, bias_type: int = 0) -> int:
        """Registers an extra epilogue record (raw pointers) and returns its index for ``per_tile``'s ``epi``.
        ``aux_slots`` = (count, index to leave out or 15, rows between slots): mode "residual" adds every slot
        ``aux_ptr + s * rows * ld_aux`` instead of the single ``aux`` block. Mode "scatter_rows": ``aux_ptr`` is the
        table of 16-byte {token, k, weight} row records and ``bias_type`` the number of k slots per token
        (MACO_EPI_SCATTER_ROWS in csrc/maco_types.h)."""
        pack = 0
        if aux_slots is not None:
            cnt, skip, rows = aux_slots
            if not (2 <= cnt <= 15 and 0 <= skip <= 15 and 0 <= rows < (1 << 23)):
                raise ValueError("aux_slots: 2..15 slots, skip index 0..15, fewer than 2^23 rows between slots")
            pack = cnt | (skip << 4) | (rows << 8)
        self.epis.append(_pack_epilogue(out_ptr, 0, aux_ptr, ld_out, ld_aux, EPI[mode], N.DTYPE_CODE[out_dtype], int(bias_type),
                                        N.DTYPE_CODE[aux_dtype] if aux_dtype is not None else 0, M, Nn, float(alpha), pack))
        return len(self.epis) - 1

    def gemm(self, a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor], *, trans_a: bool = False,
             trans_b: bool = False, epilogue: Optional[str] = None, bias: Optional[torch.Tensor] = None,
             aux: Optional[torch.Tensor] = None, alpha: float = 1.0, bn: int = 0,
             a_ready: Optional[RowEvents] = None, extra_waits: Sequence[Tuple[int, int, bool, bool]] = (),
             per_tile=None, m_blocks: Optional[Sequence[int]] = None, signal_sys: bool = False,
             row_wait=None, group_blocks: Optional[int] = None) -> RowEvents:
        """Adds the tiles of ``out = epilogue(alpha * A · B^T)`` (A logically [M,K], B logically [N,K]).

        ``a_ready`` gives row-block events of A (a tile waits only for its 128 rows); ``extra_waits``
        apply to every tile. ``per_tile(mb, nb) -> dict`` may override ``peer``, ``out_off``,
        ``row_off``, ``signal_peer``, ``signal_peer_event``, ``epi`` (index from ``add_epilogue``) and add
        ``waits`` per tile (fused GEMM -> reduce-scatter).
        ``row_wait(mb) -> wait`` supplies a per-row-block wait instead of ``a_ready``.
        ``group_blocks``: tiles are emitted as groups of that many row blocks sweeping all column tiles. While a
        group runs, its A panel (group_blocks x 128 x K) stays in L2 and B streams through once, so DRAM reads
        B once per GROUP: large groups cut the re-reads of a B that does not fit the 126 MB L2. Default: as many
        blocks as keep the A panel near 32 MB (MACO_GEMM_PANEL_MB; at least 8) when the caller did not fix the block order, else 8.
        """
        for t in (a, b):
            if t.dim() != 2 or t.stride(1) != 1 or t.dtype not in (torch.bfloat16, torch.float16):
                raise ValueError("tcgen05 GEMM tasks need row-major 2-D bf16/fp16 operands")
            if t.data_ptr() % 16 or (t.stride(0) * 2) % 16:
                raise ValueError("tcgen05 GEMM tasks need 16-byte aligned operand rows")
        M, K = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
        Nn, Kb = (b.shape[1], b.shape[0]) if trans_b else (b.shape[0], b.shape[1])
        if K != Kb:
            raise ValueError("inner dimensions differ")
        mode = EPI[epilogue]
        if bn == 0:
            m_tiles = (M + BM - 1) // BM
            # the SwiGLU epilogue needs the weight interleaved for the tile width; 256 unless told otherwise
            bn = 128 if (Nn <= 128 or (m_tiles * ((Nn + 255) // 256) < self.num_workers and mode != 2)) else 256
        if bn not in (128, 256):
            raise ValueError("bn must be 128 or 256")
        ab = 1 if a.dtype == torch.bfloat16 else 0
        pair = self.cta_pair
        # two-CTA tiles: the instruction spans 256 rows (two row blocks) and each CTA loads bn/2 rows of B
        idesc = make_idesc(ab, 2 * BM if pair else BM, bn, int(trans_a), int(trans_b))
        ta = self._tmap(a, a.shape[0], a.shape[1], a.stride(0), trans_a, BM)
        tb = self._tmap(b, b.shape[0], b.shape[1], b.stride(0), trans_b, bn // 2 if pair else bn)
        out_ptr = out.data_ptr() if out is not None else 0
        ld_out = out.stride(0) if out is not None else 0
        out_type = N.DTYPE_CODE[out.dtype] if out is not None else N.DTYPE_CODE[a.dtype]
        self.epis.append(_pack_epilogue(out_ptr, N.ptr(bias), N.ptr(aux), ld_out, aux.stride(0) if aux is not None else 0,
                                        mode, out_type, N.DTYPE_CODE[bias.dtype] if bias is not None else 0,
                                        N.DTYPE_CODE[aux.dtype] if aux is not None else 0, M, Nn, float(alpha)))
        epi = len(self.epis) - 1
        if epi > 0xFFFF or len(self.tmaps) > 0xFFFF:
            raise ValueError("too many epilogues / tensor maps in one program")
        self.keepalive += [t for t in (a, b, out, bias, aux) if t is not None]
        node_id = self.new_node_id()
        m_tiles, n_tiles, k_blocks = (M + BM - 1) // BM, (Nn + bn - 1) // bn, (K + BK - 1) // BK
        mbs = list(m_blocks) if m_blocks is not None else list(range(m_tiles))
        all_ev = self.new_event()
        row_events = {mb: self.new_event() for mb in mbs}
        base_waits = self.join(list(extra_waits), node_id)

        def tile_waits(mb: int) -> list:
            waits = list(base_waits)
            if row_wait is not None:
                w = row_wait(mb)
                if w is not None:
                    waits.append(w)
            elif a_ready is not None:
                ev, cnt = a_ready.for_rows(mb * BM, min(M, (mb + 1) * BM))
                waits.append((ev, cnt, a_ready.sys, False))
            waits = list(dict.fromkeys(waits))
            if len(waits) > 2:
                waits = self.join(waits, node_id)
            return waits

        def prepare(mb: int, nb: int):
            """The tile's wait conditions (reduced to two, which may add join tasks) and per-tile overrides."""
            first_join = len(self.tasks)
            waits = tile_waits(mb)
            ov = per_tile(mb, nb) if per_tile is not None else {}
            if ov.get("waits"):
                waits = list(dict.fromkeys(waits + list(ov["waits"])))
                if len(waits) > 2:
                    waits = self.join(waits, node_id)
            if pair and ov.get("count_ptr", 0):
                raise ValueError("run-time counted tiles are not available in two-CTA programs")
            return waits, ov, range(first_join, len(self.tasks))

        def emit(mb: int, nb: int, half: Optional[int], prepared=None) -> None:
            waits, ov, joins = prepared if prepared is not None else prepare(mb, nb)
            # The tile's own join tasks run on the tile's worker, directly in front of it: a join blocks the worker
            # that holds it, and on any other worker it would stall that worker's tiles (and, in two-CTA
            # programs, its partner) for a condition only this tile cares about.
            for j in joins:
                self.tasks[j]["attach_to"] = len(self.tasks)
            raw = _pack_gemm(ta, tb, ov.get("epi", epi), int(trans_a), int(trans_b), mb * BM, nb * bn, 0, k_blocks, idesc,
                             ov.get("peer", -1), ov.get("row_off", 0), ov.get("out_off", 0), bn,
                             ov.get("count_base", 0), ov.get("count_ptr", 0))
            self.add_task(int(TaskType.LINEAR), raw, waits=waits, signals=[row_events[mb], all_ev],
                          signal_peer=ov.get("signal_peer", -1), signal_peer_event=ov.get("signal_peer_event", -1),
                          node_id=node_id, signal_sys=signal_sys, counted=bool(ov.get("count_ptr", 0)), pair_half=half)

        def emit_filler(nb: int) -> None:
            # second half of a pair that has only one row block left: rows past the end of A (the loads return
            # zeros, the epilogue stores nothing), no conditions, no signals; it keeps the pair's protocol whole
            raw = _pack_gemm(ta, tb, epi, int(trans_a), int(trans_b), m_tiles * BM, nb * bn, 0, k_blocks, idesc, -1, 0, 0, bn)
            self.add_task(int(TaskType.LINEAR), raw, node_id=node_id, pair_half=1)

        if group_blocks is None:
            G = 8
            if m_blocks is None:
                import os
                panel_mb = float(os.environ.get("MACO_GEMM_PANEL_MB", "32"))
                G = max(8, min(len(mbs), int(panel_mb * (1 << 20)) // max(1, BM * K * a.element_size())))
        else:
            G = max(1, int(group_blocks))
        G += G & 1 if self.cta_pair else 0           # whole pairs of row blocks per group
        for g0 in range(0, len(mbs), G):
            grp = mbs[g0:g0 + G]
            # tiles of `G` row blocks sweep all column tiles: operands stay in L2, row blocks finish in order
            for nb in range(n_tiles):
                if not pair:
                    for mb in grp:
                        emit(mb, nb, None)
                    continue
                for j in range(0, len(grp), 2):
                    # Join tasks of BOTH halves go in front of both halves: the leader half cannot finish before
                    # the other half's operands are loaded, so nothing the other half waits for may sit behind the
                    # leader half in any queue (static queues follow emission order).
                    p0 = prepare(grp[j], nb)
                    p1 = prepare(grp[j + 1], nb) if j + 1 < len(grp) else None
                    emit(grp[j], nb, 0, p0)
                    if p1 is not None:
                        emit(grp[j + 1], nb, 1, p1)
                    else:
                        emit_filler(nb)
        total = len(mbs) * n_tiles
        return RowEvents(rows=M, block=BM, row_events=[(row_events.get(mb, all_ev), n_tiles) if mb in row_events
                                                       else (all_ev, total) for mb in range(m_tiles)],
                         all_event=(all_ev, total), sys=signal_sys)

    def _emit_groups(self) -> None:
        """Dispatch groups of the scheduler CTA: maximal runs of consecutive tasks with identical wait
        conditions and worker class (so a group becomes ready as a whole)."""
        self.groups = []
        i, n = 0, len(self.tasks)
        mask = TF_WAIT0_SYS | TF_WAIT1_SYS | TF_COMM_WORKER | TF_WAIT0_PREV | TF_WAIT1_PREV

        def key(t):
            return (tuple(t["wait_event"]), tuple(t["wait_count"]), t["flags"] & mask)

        while i < n:
            k = key(self.tasks[i])
            j = i + 1
            while j < n and key(self.tasks[j]) == k:
                j += 1
            t = self.tasks[i]
            self.groups.append(dict(first_task=i, num_tasks=j - i, wait_event=list(t["wait_event"]),
                                    wait_count=list(t["wait_count"]), flags=t["flags"] & mask))
            i = j

    # ------------------------------------------------------------------ split-K GEMM for few rows (decode)
    def gemm_splitk(self, a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], *, split_k: int = 0,
                    epilogue: Optional[str] = None, aux: Optional[torch.Tensor] = None,
                    a_ready: Optional[RowEvents] = None, extra_waits: Sequence[Tuple[int, int, bool, bool]] = (),
                    heap_out_off: Optional[int] = None, ld_out: Optional[int] = None,
                    signal_peer_event: int = -1, rows_per_task: int = 0, fused_finish: Optional[bool] = None,
                    w_blocked: Optional[torch.Tensor] = None, rope: Optional[dict] = None) -> RowEvents:
        """``out = op(a @ w.T)`` for at most 128 rows, bound by streaming ``w`` out of HBM.

        The K dimension is cut into ``split_k`` slices (0: enough slices for every worker to hold a tile),
        256-column tcgen05 tiles add their fp32 partial sums into one workspace with vector reductions,
        and a finishing pass (csrc/splitk_tasks.cuh) applies ``epilogue`` (None, "swiglu" over the
        interleaved gate/up layout, "residual" with ``aux``) and writes the 16-bit result: into ``out``, or,
        with ``heap_out_off``, at that byte offset of EVERY rank's symmetric heap (the exchange step of a
        one-shot all-reduce), bumping ``signal_peer_event`` on every rank.
        ``epilogue="qk_rope"`` (a fused QKV projection, head_dim 128; needs ``rope`` = dict(q_out [M, hq, 128],
        k_cache, v_cache [M, hkv, S, 128], q_norm, k_norm [128], cos_sin [M, 128], hq, hkv, pos, eps) and ``out=None``):
        the finishing pass applies the per-head RMSNorm and RoPE to the query and key heads and writes queries to
        ``q_out`` and keys / values straight into row ``pos`` of their caches (MacoQkRopeParams in csrc/maco_types.h);
        no QKV buffer and no separate QK-norm + RoPE tasks. Fused finishing only.
        ``w_blocked``: the same weight laid out tile by tile (``ops.block_weight(w)``, [N/256, K/64, 256, 64]); the
        tiles then load contiguous 32 KB blocks (``w`` itself is not read).
        ``fused_finish`` (default: on for a local ``out``, off with ``heap_out_off``; env ``MACO_SPLITK_FUSED=0``
        turns it off): the tile that arrives last at
        its column tile's counter runs the finishing pass for those columns in its own epilogue warps, while the
        worker's TMA and MMA warps stream the next tile. Off: SPLITK_FIN tasks behind an event that counts all
        tiles (one more dependency hop and a tail of short tasks).
        The reference runs such GEMMs as one torch.mm each (maco/task_graph/runtime.py:188-209).
        """
        if self.cta_pair:
            raise ValueError("split-K GEMMs are not available in two-CTA programs")
        M, K = a.shape
        Nn = w.shape[0]
        if M > BM or w.shape[1] != K or Nn % 256 or K % BK:
            raise ValueError("gemm_splitk: at most 128 rows, N a multiple of 256, K a multiple of 64")
        mode = {None: 0, "none": 0, "swiglu": 1, "residual": 2, "qk_rope": 3}[epilogue]
        rope_dev = None
        if mode == 3:
            if rope is None or out is not None or heap_out_off is not None or fused_finish is False:
                raise ValueError("gemm_splitk: epilogue 'qk_rope' takes rope=..., out=None, a local result and fused finishing")
            hq, hkv = int(rope["hq"]), int(rope["hkv"])
            q_out, kc, vc = rope["q_out"], rope["k_cache"], rope["v_cache"]
            if Nn != (hq + 2 * hkv) * 128 or kc.shape[-1] != 128 or kc.dim() != 4 or kc.shape[1] != hkv or not kc.is_contiguous() \
                    or not vc.is_contiguous() or vc.shape != kc.shape or tuple(q_out.shape) != (M, hq, 128) or not q_out.is_contiguous() \
                    or rope["cos_sin"].shape != (M, 128) or not (0 <= int(rope["pos"]) < kc.shape[2]):
                raise ValueError("gemm_splitk: rope tensors do not match (hq + 2 hkv) heads of 128 and caches [M, hkv, S, 128]")
            fused_finish = True
            blob = struct.pack("<QQQQQQqqiiiifi", q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), rope["q_norm"].data_ptr(),
                               rope["k_norm"].data_ptr(), rope["cos_sin"].data_ptr(), kc.stride(0), kc.stride(1), hq, hkv,
                               int(rope["pos"]), N.DTYPE_CODE[q_out.dtype], float(rope["eps"]), 0)
            rope_dev = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(a.device)
            self.keepalive += [rope_dev, q_out, kc, vc, rope["q_norm"], rope["k_norm"], rope["cos_sin"]]
        n_tiles, k_blocks = Nn // 256, K // BK
        if split_k <= 0:
            split_k = pick_split_k(n_tiles, k_blocks, self.num_workers)
        split_k = max(1, min(split_k, k_blocks))
        ws = torch.zeros(M, Nn, device=a.device, dtype=torch.float32)      # SPLITK_FIN leaves it zeroed again
        self.launch_state.append(ws)
        out_dtype = out.dtype if out is not None else a.dtype
        ab = 1 if a.dtype == torch.bfloat16 else 0
        idesc = make_idesc(ab, BM, 256, 0, 0)
        ta = self._tmap(a, a.shape[0], a.shape[1], a.stride(0), False, BM)
        if w_blocked is not None:
            if tuple(w_blocked.shape) != (n_tiles, k_blocks, 256, BK) or not w_blocked.is_contiguous() or w_blocked.dtype != w.dtype:
                raise ValueError("gemm_splitk: w_blocked must be ops.block_weight(w) ([N/256, K/64, 256, 64], contiguous)")
            tb = self._tmap(w_blocked.view(-1, BK), n_tiles * k_blocks * 256, BK, BK, False, 256)
            self.keepalive.append(w_blocked)
        else:
            tb = self._tmap(w, w.shape[0], w.shape[1], w.stride(0), False, 256)
        out_cols = Nn // 2 if mode == 1 else Nn
        ld_o = ld_out if ld_out is not None else (out.stride(0) if out is not None else out_cols)
        if aux is not None and aux.stride(0) != ld_o:
            raise ValueError("gemm_splitk: aux must have the output's row stride")
        dt = N.DTYPE_CODE[out_dtype]
        es = 2
        if fused_finish is None:
            import os
            # A result that goes into every rank's heap is finished by tasks spread over all workers: with the
            # fused form only the last arrival of each 256-column tile (20 CTAs for 5120 columns) would push all
            # rows to every peer (measured: the 4-GPU decode layer's o-proj ended 35 us later).
            fused_finish = os.environ.get("MACO_SPLITK_FUSED", "1") != "0" and heap_out_off is None
        if fused_finish:
            # the tile that arrives last at its column tile's counter finishes those columns itself
            # (MACO_EPI_SPLITK_FUSED in csrc/maco_types.h): no finishing tasks, no hop between the two halves
            counters = torch.zeros(n_tiles, device=a.device, dtype=torch.int32)
            self.launch_state.append(counters)
            fin = _pack_elt(ws.data_ptr(), rope_dev.data_ptr() if rope_dev is not None else (aux.data_ptr() if aux is not None else 0),
                            heap_out_off or 0,
                            out.data_ptr() if out is not None else 0, 0, M, out_cols, dt, Nn, ld_o, i0=mode,
                            i1=-2 if heap_out_off is not None else -1)
            fin_dev = torch.frombuffer(bytearray(fin), dtype=torch.uint8).to(a.device)
            self.keepalive += [counters, fin_dev]
            self.epis.append(_pack_epilogue(ws.data_ptr(), counters.data_ptr(), fin_dev.data_ptr(), Nn, 0, EPI["splitk_fused"],
                                            N.DTYPE_CODE[torch.float32], split_k, 0, M, Nn, 1.0))
        else:
            self.epis.append(_pack_epilogue(ws.data_ptr(), None, None, Nn, 0, EPI["f32_atomic"], N.DTYPE_CODE[torch.float32], 0, 0,
                                            M, Nn, 1.0))
        epi = len(self.epis) - 1
        self.keepalive += [t for t in (a, w, out, aux, ws) if t is not None]
        node_id = self.new_node_id()
        waits = list(extra_waits)
        if a_ready is not None:
            ev, cnt = a_ready.for_rows(0, M)
            waits.append((ev, cnt, a_ready.sys, False))
        waits = self.join(list(dict.fromkeys(waits)), node_id)
        e_ws = self.new_event()
        n_parts = 0
        for sp in range(split_k):
            kb0 = sp * k_blocks // split_k
            kb1 = (sp + 1) * k_blocks // split_k
            for nb in range(n_tiles):
                # b_mn bit 1 + count_base: blocked B and its total number of k-blocks (csrc/maco_types.h)
                raw = _pack_gemm(ta, tb, epi, 0, 2 if w_blocked is not None else 0, 0, nb * 256, kb0 * BK, kb1 - kb0, idesc,
                                 -1, 0, 0, 256, count_base=k_blocks if w_blocked is not None else 0)
                if fused_finish:
                    self.add_task(int(TaskType.LINEAR), raw, waits=waits, signals=[e_ws], node_id=node_id,
                                  signal_peer=-2 if signal_peer_event >= 0 else -1, signal_peer_event=signal_peer_event)
                else:
                    self.add_task(int(TaskType.LINEAR), raw, waits=waits, signals=[e_ws], node_id=node_id)
                n_parts += 1
        if fused_finish:
            return RowEvents(rows=M, block=BM, row_events=[(e_ws, n_parts)], all_event=(e_ws, n_parts))
        # second half: one task per few rows, spread over the workers
        if rows_per_task <= 0:
            rows_per_task = max(1, M // self.num_workers)
        # one task per (row group, column chunk): about one per worker (a task costs several us of fixed
        # latency: descriptor, dependency check, store drain, signal), chunks whole 128-column blocks
        n_rowtasks = -(-M // rows_per_task)
        chunks = max(1, min(out_cols // 128, self.num_workers // n_rowtasks))
        while out_cols % (chunks * 128):
            chunks -= 1
        nc = out_cols // chunks
        done = self.new_event()
        n_fin = 0
        for r0 in range(0, M, rows_per_task):
            rr = min(rows_per_task, M - r0)
            for ch in range(chunks):
                c0 = ch * nc
                ws_c0 = (c0 // 128) * 256 if mode == 1 else c0
                raw = _pack_elt(ws.data_ptr() + ws_c0 * 4, aux.data_ptr() + c0 * es if aux is not None else 0,
                                heap_out_off + c0 * es if heap_out_off is not None else 0,
                                out.data_ptr() + c0 * es if out is not None else 0,
                                r0, rr, nc, dt, Nn, ld_o, i0=mode, i1=-2 if heap_out_off is not None else -1)
                self.add_task(T_SPLITK_FIN, raw, waits=[(e_ws, n_parts, False, False)], signals=[done],
                              signal_peer=-2 if signal_peer_event >= 0 else -1, signal_peer_event=signal_peer_event,
                              node_id=node_id)
                n_fin += 1
        return RowEvents(rows=M, block=BM, row_events=[(done, n_fin)], all_event=(done, n_fin))

    # ------------------------------------------------------------------ decode attention node
    def attention_decode(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor, *,
                         kv_len: Optional[int] = None, splits: int = 1, scale: Optional[float] = None,
                         waits: Sequence[Tuple[int, int, bool, bool]] = (), balance: bool = False) -> Tuple[int, int]:
        """Split-KV decode attention: q [B, hq, D] against caches [B, hkv, S, D] -> out [B, hq, D].

        One ATTENTION task per (sequence, kv head, split) writes an fp32 partial {o, m, l}. 16-bit caches
        run on the tensor cores (csrc/attention_decode.cuh), fed by TMA through tensor maps over the
        flattened caches, and the split that finishes last for a (sequence, kv head) combines the records
        itself; other element types use the CUDA-core task plus one ATTN_MERGE task per (sequence, kv
        head), emitted after all attention tasks (with static queues a merge placed right behind its
        splits would hold its worker idle until the neighbours finish theirs).
        Returns (event, count) that is complete when every output row is final.
        The reference declares ATTENTION as a task type and never implements it (maco/csrc/maco_types.h:24-40).
        """
        if self.cta_pair:
            raise ValueError("attention tasks are not available in two-CTA programs")
        B, hq, D = q.shape
        _, hkv, S, _ = k_cache.shape
        G = hq // hkv
        kv_len = S if kv_len is None else kv_len
        if hq % hkv or G > 8 or D != 128 or kv_len > S:
            raise ValueError("attention_decode: head_dim 128, at most 8 query heads per kv head, kv_len <= cache length")
        if not (q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous() and out.is_contiguous()):
            raise ValueError("attention_decode: contiguous tensors only")
        dt = N.DTYPE_CODE[q.dtype]
        es = q.element_size()
        scale = D ** -0.5 if scale is None else scale
        rec = G * D + 2 * G
        partials = torch.empty(B * hkv * splits * rec, device=q.device, dtype=torch.float32)
        self.keepalive += [q, k_cache, v_cache, out, partials]
        tm_kv = 0
        if es == 2:
            rows_total = B * hkv * S
            tk = self._tmap(k_cache.view(rows_total, D), rows_total, D, D, False, BM)
            tv = self._tmap(v_cache.view(rows_total, D), rows_total, D, D, True, 64)
            tm_kv = (tk + 1) | ((tv + 1) << 16)
        waits = self.join(list(waits))
        per = -(-kv_len // splits)
        splits = -(-kv_len // per)                         # every split holds at least one key
        merged = self.new_event()
        if tm_kv:
            # tensor-core path: the split that finishes last for a (sequence, kv head) merges the records itself.
            # Pieces: either `splits` equal parts per (sequence, kv head), or (balance) the whole key range cut
            # into one equal share per worker at 128-key boundaries, so no worker runs an extra wave.
            pieces = []                                     # (bh, first key, keys, worker or None)
            if balance:
                pieces = attention_pieces(B * hkv, kv_len, self.num_workers)
            else:
                for bh in range(B * hkv):
                    for sp in range(splits):
                        pieces.append((bh, sp * per, min(per, kv_len - sp * per), None))
            n_of = [0] * (B * hkv)
            for bh, _, _, _ in pieces:
                n_of[bh] += 1
            partials = torch.empty(len(pieces) * rec, device=q.device, dtype=torch.float32)
            counters = torch.zeros(B * hkv, device=q.device, dtype=torch.int32)   # only ever grow: one per piece and launch
            self.keepalive += [partials, counters]
            self.launch_state.append(counters)
            idx_in_group = [0] * (B * hkv)
            for pi, (bh, s0, keys, wk) in enumerate(pieces):
                bi, j = divmod(bh, hkv)
                sp = idx_in_group[bh]
                idx_in_group[bh] += 1
                row = (bi * hkv + j) * S + s0
                # records of a group are consecutive: the piece index minus its position is the group's first record
                raw = _pack_elt(q.data_ptr() + (bi * hq + j * G) * D * es, counters.data_ptr() + bh * 4,
                                out.data_ptr() + (bi * hq + j * G) * D * es, partials.data_ptr() + pi * rec * 4,
                                row, keys, D, dt, D, tm_kv, f0=scale, f1=float(sp), i0=G, i1=n_of[bh])
                self.add_task(int(TaskType.ATTENTION), raw, waits=waits, signals=[merged], worker=wk)
            return merged, len(pieces)
        merges = []
        for bh in range(B * hkv):
            bi, j = divmod(bh, hkv)
            ev = self.new_event()
            n_split = 0
            for sp in range(splits):
                s0 = sp * per
                keys = max(0, min(per, kv_len - s0))
                row = (bi * hkv + j) * S + s0
                raw = _pack_elt(q.data_ptr() + (bi * hq + j * G) * D * es, k_cache.data_ptr() + row * D * es,
                                v_cache.data_ptr() + row * D * es, partials.data_ptr() + (bh * splits + sp) * rec * 4,
                                row, keys, D, dt, D, 0, f0=scale, i0=G)
                self.add_task(int(TaskType.ATTENTION), raw, waits=waits, signals=[ev])
                n_split += 1
            raw = _pack_elt(partials.data_ptr() + bh * splits * rec * 4, 0, 0, out.data_ptr() + (bi * hq + j * G) * D * es,
                            0, 0, D, dt, 0, 0, i0=G, i1=splits)
            merges.append((raw, ev, n_split))
        for raw, ev, n_split in merges:
            self.add_task(int(TaskType.ATTN_MERGE), raw, waits=[(ev, n_split, False, False)], signals=[merged])
        return merged, B * hkv

    # ------------------------------------------------------------------ element-wise / row-wise node
    def elementwise(self, ttype: int, in0: torch.Tensor, out: torch.Tensor, *, in1: Optional[torch.Tensor] = None,
                    in2: Optional[torch.Tensor] = None, rows: int, cols: int, f0: float = 0.0, f1: float = 0.0,
                    i0: int = 0, i1: int = 0, in_ready: Sequence[Optional[RowEvents]] = (),
                    extra_waits: Sequence[Tuple[int, int, bool, bool]] = (), rows_per_task: Optional[int] = None,
                    ld_in: Optional[int] = None, ld_out: Optional[int] = None, all_event: Optional[int] = None) -> RowEvents:
        """Row-chunked task list for an operator of csrc/elementwise.cuh over a [rows, cols] view.
        ``all_event`` lets several calls bump one shared completion event (the caller adds up the counts),
        so that a consumer of all of them needs one wait condition instead of a chain of joins."""
        dt = N.DTYPE_CODE[in0.dtype]
        esz = in0.element_size()
        if (ttype == int(TaskType.RMSNORM) and rows_per_task is None and i1 == 0 and rows <= self.num_workers
                and cols <= 8192 and cols % 8 == 0):
            rows_per_task, i1 = 1, 1      # decode: one row per task, all 128 threads of the worker on it
        if rows_per_task is None:
            target = max(1, (256 * 1024) // max(1, cols * esz))       # ~256 KiB of input per task
            if rows * cols * esz <= (4 << 20):
                # small operands (decode): latency matters more than per-task overhead; spread the rows over
                # as many workers as there are, one row per warp for the row-wise operators
                target = min(target, max(4 if ttype in (103, 104, 107) else 1, -(-rows // self.num_workers)))
            rows_per_task = 1
            while rows_per_task * 2 <= min(target, BM):
                rows_per_task *= 2
        self.keepalive += [t for t in (in0, in1, in2, out) if t is not None]
        node_id = self.new_node_id()
        all_ev = self.new_event() if all_event is None else all_event
        n_blocks = (rows + BM - 1) // BM
        row_events = [self.new_event() for _ in range(n_blocks)]
        counts = [0] * n_blocks
        base_waits = self.join(list(extra_waits), node_id)
        total = 0
        for r0 in range(0, rows, rows_per_task):
            r1 = min(rows, r0 + rows_per_task)
            waits = list(base_waits)
            for re_ in in_ready:
                if re_ is not None:
                    ev, cnt = re_.for_rows(r0, r1) if re_.rows == rows else re_.all_event
                    waits.append((ev, cnt, re_.sys, False))
            waits = list(dict.fromkeys(waits))
            if len(waits) > 2:
                waits = self.join(waits, node_id)
            raw = _pack_elt(in0.data_ptr(), N.ptr(in1), N.ptr(in2), out.data_ptr(), r0, r1 - r0, cols, dt,
                            ld_in if ld_in is not None else cols, ld_out if ld_out is not None else cols, f0, f1, i0, i1)
            blk = r0 // BM
            self.add_task(ttype, raw, waits=waits, signals=[row_events[blk], all_ev], node_id=node_id)
            counts[blk] += 1
            total += 1
        return RowEvents(rows=rows, block=BM, row_events=list(zip(row_events, counts)), all_event=(all_ev, total))

    # ------------------------------------------------------------------ build
    def build(self) -> "Program":
        self._emit_groups()
        return Program(self)


class DescriptorError(ValueError):
    """A task descriptor points outside the tables or the heap it may touch (found when the program is built)."""


def validate_tasks(b: "ProgramBuilder") -> None:
    """Host-side check of every descriptor: event, tensor-map and epilogue indices inside their tables, peer ranks
    inside the world, and every block a communication task or a GEMM tile writes into (or reads from) a PEER's
    heap inside the heap. The kernel repeats the same checks per task when ``config.debug`` is set."""
    n_ev, n_tm, n_ep = max(1, b.num_events), len(b.tmaps), len(b.epis)
    world = b.heap.world if b.heap is not None else 1
    heap_bytes = b.heap.nbytes if b.heap is not None else 0
    for i, t in enumerate(b.tasks):
        def bad(msg):
            raise DescriptorError(f"task {i} (type {t['type']}): {msg}")
        for e in list(t["wait_event"]) + list(t["signal_event"]) + [t["signal_peer_event"]]:
            if e >= n_ev:
                bad(f"event {e} outside the table of {n_ev}")
        if t["signal_peer"] >= world or t["signal_peer"] < -4:
            bad(f"signal_peer {t['signal_peer']} outside the world of {world}")
        raw = t["raw"]
        if t["type"] in (100, 101) and len(raw) >= 60:
            tm_a, tm_b, epi, _, _, _, _, _, k_blocks, _, peer, _, out_off, bn = struct.unpack_from("<HHHBBiiiiIiqQI", raw)
            if tm_a >= n_tm or tm_b >= n_tm or epi >= n_ep:
                bad("tensor-map or epilogue index outside its table")
            if peer >= world or peer < -2:
                bad(f"destination rank {peer} outside the world of {world}")
            if peer != -1 and out_off >= heap_bytes:
                bad(f"tile destination offset {out_off} outside the heap of {heap_bytes} bytes")
            if bn not in (128, 256) or k_blocks < 0:
                bad("bad tile width or k-block count")
        elif 200 <= t["type"] < 300 and len(raw) >= 72:
            src_off, dst_off, s_str, d_str, row_bytes, rows, _, peer, op, _, _, local_ptr = struct.unpack_from("<QQQQIIiiiiQQ", raw)
            if rows == 0:
                continue
            if row_bytes % 16:
                bad("rows must be whole 16-byte vectors")
            if peer >= world or peer < -3:
                bad(f"peer {peer} outside the world of {world}")
            ext = (rows - 1) * d_str + row_bytes
            if local_ptr == 0 and op != COMM_REDUCE_LOCAL and dst_off + ext > heap_bytes:
                bad(f"destination block [{dst_off}, {dst_off + ext}) outside the heap of {heap_bytes} bytes")
            if op in (COMM_REDUCE_PULL, COMM_ALLREDUCE, COMM_PULL, COMM_ALLREDUCE_MC) and src_off + (rows - 1) * s_str + row_bytes > heap_bytes:
                bad("source block read from peers lies outside the heap")
            if op in (COMM_PUSH_MC, COMM_ALLREDUCE_MC) and not (b.heap is not None and b.heap.multicast_base()):
                bad("multimem task without a multicast-bound heap")


class Program:
    """Device tables of a built program plus the launch call."""

    def __init__(self, b: ProgramBuilder):
        lib = _lib()
        validate_tasks(b)
        self.device = b.device
        self.mode = b.mode
        self.num_workers = b.num_workers
        self.num_comm_workers = b.num_comm_workers
        self.keepalive = b.keepalive
        self.launch_state = list(getattr(b, "launch_state", []))
        self.heap = b.heap
        n = len(b.tasks)
        self.num_tasks = n
        tasks = np.zeros(max(n, 1), dtype=TASK_DTYPE)
        for i, t in enumerate(b.tasks):
            rec = tasks[i]
            rec["type"], rec["flags"], rec["node_id"] = t["type"], t["flags"], t["node_id"]
            rec["wait_event"], rec["wait_count"], rec["signal_event"] = t["wait_event"], t["wait_count"], t["signal_event"]
            rec["signal_peer"], rec["signal_peer_event"] = t["signal_peer"], t["signal_peer_event"]
            raw = t["raw"]
            rec["raw"][: len(raw)] = np.frombuffer(raw, dtype=np.uint8)
        self._tasks_np = tasks
        self.task_types = tasks["type"].copy()
        dev = self.device

        def up(arr: np.ndarray) -> torch.Tensor:
            return torch.from_numpy(arr.view(np.uint8).reshape(-1).copy()).to(dev)

        self.d_tasks = up(tasks)
        self.d_tmaps = up(np.frombuffer(b"".join(b.tmaps) or bytes(128), dtype=np.uint8))
        self.d_epis = up(np.frombuffer(b"".join(b.epis) or bytes(72), dtype=np.uint8))
        groups = np.zeros(max(len(b.groups), 1), dtype=GROUP_DTYPE)
        for i, g in enumerate(b.groups):
            rec = groups[i]
            rec["first_task"], rec["num_tasks"] = g["first_task"], g["num_tasks"]
            rec["wait_event"], rec["wait_count"], rec["flags"] = g["wait_event"], g["wait_count"], g["flags"]
        self.num_groups = len(b.groups)
        self.d_groups = up(groups)
        # events live in the symmetric heap when peers must reach them
        self.num_events = max(1, b.num_events)
        if b.heap is not None:
            # Not cleared here: heap memory is zero from creation, a freed range is zeroed before it can be
            # handed out again (SymmetricHeap.free), and a peer that built this program earlier may already
            # have bumped these counters.
            self.d_events = b.heap.alloc((self.num_events + 64,), torch.int32)
        else:
            self.d_events = torch.zeros(self.num_events + 64, dtype=torch.int32, device=dev)
        self.d_ctrl = torch.zeros(8, dtype=torch.int32, device=dev)        # [0] abort word, [1] task counter
        W = self.num_workers
        queues = assign_static_queues(b.tasks, self.num_workers, self.num_comm_workers)
        from ..config import config as _dbg_cfg
        if _dbg_cfg.debug and b.heap is None and self.mode == MODE_STATIC:
            # debug layer: run the queues on the host first; an order that can deadlock is reported here, with the
            # stuck tasks, instead of as a device-side wait that runs out (single-rank programs: nothing to wait
            # for on a peer)
            simulate_static_queues([(b.tasks, queues)])
        stride = max(1, max(len(q) for q in queues))
        sq = np.full((W, stride), QUEUE_TERMINATE, dtype=np.uint32)
        for w, q in enumerate(queues):
            sq[w, : len(q)] = q
            # entries behind the queue's last ring user (GEMM tiles, pipelined attention) carry bit 31: the
            # worker's operand ring is idle from there on, and communication tasks may stage bulk copies in it
            last_gemm = max((k for k, t in enumerate(q) if b.tasks[t]["type"] in (100, 101, 102)), default=-1)
            sq[w, last_gemm + 1: len(q)] |= np.uint32(0x80000000)
        self.static_stride = stride
        self.d_static_queue = up(sq)
        self.d_static_count = up(np.array([len(q) for q in queues], dtype=np.uint32))
        if self.mode == MODE_DYNAMIC:
            self.d_ring = torch.zeros(W * WORKER_QUEUE_SIZE, dtype=torch.int32, device=dev)
            self.d_heads = torch.zeros(W, dtype=torch.int32, device=dev)
            self.d_tails = torch.zeros(W, dtype=torch.int32, device=dev)
        else:
            self.d_ring = self.d_heads = self.d_tails = None
        self.d_trace = torch.zeros(max(n, 1) * TRACE_DTYPE.itemsize, dtype=torch.uint8, device=dev) if b.trace else None
        self.epoch = 0
        ps = _ProgramStruct()
        ps.tasks, ps.tmaps, ps.epis = self.d_tasks.data_ptr(), self.d_tmaps.data_ptr(), self.d_epis.data_ptr()
        ps.events = self.d_events.data_ptr()
        ps.static_queue, ps.static_count = self.d_static_queue.data_ptr(), self.d_static_count.data_ptr()
        if self.mode == MODE_DYNAMIC:
            ps.ring, ps.heads, ps.tails = self.d_ring.data_ptr(), self.d_heads.data_ptr(), self.d_tails.data_ptr()
        ps.groups = self.d_groups.data_ptr()
        ps.abort_word = self.d_ctrl.data_ptr()
        ps.counters = self.d_ctrl.data_ptr() + 4
        ps.status = None
        ps.trace = self.d_trace.data_ptr() if self.d_trace is not None else None
        ps.budget_ns = int(b.wait_budget_ms * 1e6)
        ps.num_tasks, ps.num_groups, ps.num_workers, ps.num_comm_workers = n, self.num_groups, W, self.num_comm_workers
        ps.static_stride, ps.mode, ps.epoch = stride, self.mode, 0
        ps.rank, ps.world = 0, 1
        ps.cta_group = 2 if b.cta_pair else 1
        from ..config import config as _cfg
        ps.debug = 1 if _cfg.debug else 0
        ps.heap_bytes = b.heap.nbytes if b.heap is not None else 0
        ps.num_events, ps.num_tmaps, ps.num_epis = self.num_events + 64, max(1, len(b.tmaps)), max(1, len(b.epis))
        self.cta_pair = b.cta_pair
        if b.heap is not None:
            ps.rank, ps.world = b.heap.rank, b.heap.world
            ev_off = b.heap.offset_of(self.d_events)
            for r in range(b.heap.world):
                ps.peer_heap[r] = b.heap.peer_base(r)
                ps.peer_events[r] = b.heap.peer_base(r) + ev_off
            ps.mc_heap = b.heap.multicast_base() or None
        else:
            ps.peer_heap[0] = 0
            ps.peer_events[0] = self.d_events.data_ptr()
        self._ps = ps
        self._lib = lib
        torch.cuda.synchronize(dev)

    def run(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """One launch of the persistent kernel on ``stream`` (default: the current stream)."""
        if self.num_tasks == 0:
            return
        self.epoch += 1
        self._ps.epoch = self.epoch
        rc = self._lib.maco_program_launch(ctypes.byref(self._ps), N.current_stream_ptr(stream))
        N.check(rc, "maco_program_launch")

    def free_heap(self) -> None:
        """Gives the program's event counters back to the symmetric heap. The program must not run again.
        Collective: see ``SymmetricHeap.free``."""
        if self.heap is not None and self.d_events is not None and hasattr(self.heap, "free"):
            self.heap.free(self.d_events)
            for buf in getattr(self, "heap_buffers", []):
                self.heap.free(buf)
            self.heap_buffers = []
        self.d_events = None
        self.num_tasks = 0

    def reset_after_failure(self) -> None:
        """Re-zeroes the control state after an aborted launch (events restart from epoch 0), together with the
        buffers a launch expects in their start-of-launch state (split-K workspaces, the arrival counters of the
        tensor-core attention tasks), which an aborted launch may have left half advanced. For a program over a
        symmetric heap every rank calls this between two host barriers (the callers' job): peers bump these
        counters too."""
        torch.cuda.synchronize(self.device)
        for t in getattr(self, "launch_state", []):
            t.zero_()
        self.d_events.zero_()
        self.d_ctrl.zero_()
        if self.mode == MODE_DYNAMIC:
            self.d_heads.zero_(); self.d_tails.zero_()
        self.epoch = 0
        N.status(clear=True)

    def event_signal(self, event: int):
        """The counter behind one of the program's events as a ``DeviceSignal``: tasks bump it with release
        semantics when they finish; after launch number E it holds E times the event's per-launch count. Lets
        host code (tests, debugging, a polling thread) observe progress inside a running launch."""
        from ..sync.signal_wait import DeviceSignal
        if not 0 <= event < self.num_events:
            raise IndexError(f"event {event} outside the table of {self.num_events}")
        return DeviceSignal(self.d_events[event:event + 1])

    def tasks_completed(self) -> int:
        return int(self.d_ctrl[1].item())

    def trace_records(self) -> np.ndarray:
        if self.d_trace is None:
            return np.zeros(0, dtype=TRACE_DTYPE)
        return self.d_trace.cpu().numpy().view(TRACE_DTYPE)[: self.num_tasks]

    def stats(self) -> dict:
        rec = self.trace_records()
        if rec.size == 0:
            return {}
        rec = rec[rec["t_end_ns"] > 0]
        if rec.size == 0:
            return {}
        t0, t1 = rec["t_start_ns"].min(), rec["t_end_ns"].max()
        out = {"span_us": float(t1 - t0) / 1e3, "tasks": int(rec.size), "by_type": {}}
        for ty in np.unique(rec["type"]):
            sel = rec[rec["type"] == ty]
            name = TaskType(int(ty)).name if int(ty) in TaskType._value2member_map_ else str(int(ty))
            busy = (sel["t_end_ns"] - sel["t_start_ns"]).astype(np.float64)
            out["by_type"][name] = {"count": int(sel.size), "busy_us": float(busy.sum()) / 1e3,
                                    "wait_us": float(sel["wait_ns"].sum()) / 1e3, "mean_us": float(busy.mean()) / 1e3,
                                    "max_us": float(busy.max()) / 1e3,
                                    "first_start_us": float(sel["t_start_ns"].min() - t0) / 1e3,
                                    "last_end_us": float(sel["t_end_ns"].max() - t0) / 1e3}
        return out

    def chrome_trace(self) -> List[dict]:
        """Trace records as Chrome-trace events (one row per SM)."""
        rec = self.trace_records()
        rec = rec[rec["t_end_ns"] > 0]
        if rec.size == 0:
            return []
        t0 = int(rec["t_start_ns"].min())
        ev = []
        for r in rec:
            ty = int(r["type"])
            name = TaskType(ty).name if ty in TaskType._value2member_map_ else str(ty)
            ev.append({"name": name, "ph": "X", "pid": 0, "tid": int(r["sm"]), "ts": (int(r["t_start_ns"]) - t0) / 1e3,
                       "dur": (int(r["t_end_ns"]) - int(r["t_start_ns"])) / 1e3, "args": {"task": int(r["task"]),
                                                                                         "wait_us": int(r["wait_ns"]) / 1e3}})
        return ev

    def describe(self) -> str:
        kind = "dynamic (scheduler CTA)" if self.mode == MODE_DYNAMIC else "static queues"
        return (f"Persistent kernel: {self.num_tasks} tile tasks, {self.num_groups} dispatch groups, "
                f"{self.num_events} events, {self.num_workers} workers ({self.num_comm_workers} comm), {kind}"
                + (", two-CTA GEMM tiles" if self.cta_pair else ""))


# ---------------------------------------------------------------------------------------------------
# TaskGraph lowering
# ---------------------------------------------------------------------------------------------------
_ELT_TYPES = {TaskType.GELU, TaskType.SILU, TaskType.SOFTMAX, TaskType.SCALE, TaskType.ADD, TaskType.SILU_GATE,
              TaskType.RMSNORM, TaskType.LAYERNORM, TaskType.ROPE}
_F16 = (torch.bfloat16, torch.float16)


def _flat2d(t: torch.Tensor) -> Optional[torch.Tensor]:
    if t.dim() == 0 or not t.is_contiguous():
        return None
    return t.view(-1, t.shape[-1])


def _gemm_ok(node: TaskNode) -> bool:
    ins = node.inputs
    x, w = ins[0], ins[1]
    if x.dtype not in _F16 or w.dtype != x.dtype:
        return False
    x2 = _flat2d(x)
    if x2 is None or w.dim() != 2 or w.stride(1) != 1:
        return False
    out = node.outputs[0]
    if not out.is_contiguous():
        return False
    for t in (x2, w):
        if t.numel() and (t.data_ptr() % 16 or (t.stride(0) * 2) % 16):
            return False
    if out.numel() and (out.data_ptr() % 16 or (out.shape[-1] * 2) % 16):
        return False
    return True


def can_lower(graph) -> bool:
    """True when every node has a task form. Custom host callables, and collectives over more than one rank
    when there is no symmetric heap (or for shapes the communication tasks cannot express), are run by the
    stream runtime instead."""
    from ..comm.process_group import get_world_size
    if not graph._nodes:
        return False
    world = get_world_size()
    for n in graph._nodes:
        t = n.task_type
        if t in (TaskType.LINEAR, TaskType.MATMUL):
            if not _gemm_ok(n):
                return False
        elif t in _ELT_TYPES:
            if any(not x.is_contiguous() for x in n.inputs + n.outputs) or n.inputs[0].dtype not in N.DTYPE_CODE:
                return False
            if any(x.dtype != n.inputs[0].dtype for x in n.inputs):
                return False
        elif t == TaskType.NOP:
            pass
        elif t in (TaskType.ALLREDUCE, TaskType.BROADCAST, TaskType.ALL_TO_ALL, TaskType.ALLGATHER, TaskType.REDUCE_SCATTER):
            if any(not x.is_contiguous() for x in n.inputs + n.outputs):
                return False
            if world > 1:
                # more than one rank: the collective becomes communication tasks over the symmetric heap
                from ..parallel.graph_collectives import can_lower_collective
                from ..parallel.symm_heap import current_heap
                if not can_lower_collective(n, current_heap()):
                    return False
        else:
            return False
    return True


def lower_graph(graph, mode: Optional[str] = None, trace: Optional[bool] = None) -> Program:
    """Lowers a TaskGraph (dependencies already inferred) to a persistent-kernel program."""
    import os
    from ..config import config
    mode = mode or os.environ.get("MACO_PERSISTENT_MODE", "static")
    trace = config.profile if trace is None else trace
    sms = torch.cuda.get_device_properties(graph.device).multi_processor_count
    workers = min(graph.num_workers, sms - (1 if mode == "dynamic" else 0))

    def _few_rows(n: TaskNode) -> bool:
        x2, w = _flat2d(n.inputs[0]), n.inputs[1]
        return (n.task_type == TaskType.LINEAR and not n.attrs.get("has_bias") and n.attrs.get("activation") in (None, "none", "swiglu")
                and x2.shape[0] <= BM and w.shape[0] % 256 == 0 and x2.shape[1] % BK == 0 and w.shape[0] * w.shape[1] >= (1 << 22))

    gemm_nodes = [n for n in graph._nodes if n.task_type in (TaskType.LINEAR, TaskType.MATMUL) and n.outputs and n.outputs[0].numel()]
    # two-CTA tiles pay once the 256-row tiles of every GEMM cover the worker pairs; decode-shaped (split-K)
    # nodes keep the graph on one-CTA tiles
    cta_pair = (mode == "static" and workers >= 4 and bool(gemm_nodes) and not any(_few_rows(n) for n in gemm_nodes)
                and all(-(-_flat2d(n.inputs[0]).shape[0] // (2 * BM)) * -(-n.outputs[0].shape[-1] // 256) >= workers // 2
                        for n in gemm_nodes))
    from ..comm.process_group import get_world_size
    _COLL = (TaskType.ALLREDUCE, TaskType.BROADCAST, TaskType.ALL_TO_ALL, TaskType.ALLGATHER, TaskType.REDUCE_SCATTER)
    dist = get_world_size() > 1 and any(n.task_type in _COLL for n in graph._nodes)
    heap, comm_workers = None, 0
    if dist:
        from ..parallel.symm_heap import current_heap
        heap = current_heap()
        comm_workers = graph_comm_workers(graph, workers)
        mode = "static"
    b = ProgramBuilder(graph.device, num_workers=workers, mode=mode, trace=trace, cta_pair=cta_pair and mode == "static",
                       heap=heap, num_comm_workers=comm_workers)
    ctx = None
    fused_rs: Dict[int, TaskNode] = {}                         # linear node id -> the reduce_scatter it feeds
    skip: Dict[int, bool] = {}
    if dist:
        from ..parallel import graph_collectives as gc
        ctx = gc.DistContext(b)
        consumers: Dict[int, List[TaskNode]] = {}
        for n in graph._nodes:
            for d in n.depends_on:
                consumers.setdefault(d._node_id, []).append(n)
        for n in graph._nodes:
            cs = consumers.get(n._node_id, [])
            if (len(cs) == 1 and cs[0].task_type == TaskType.REDUCE_SCATTER and len(cs[0].depends_on) == 1
                    and gc.fusable_linear_reduce_scatter(n, cs[0], heap.world) and not _few_rows(n)):
                fused_rs[n._node_id] = cs[0]
    produced: Dict[int, Tuple[TaskNode, RowEvents]] = {}       # node id -> events of its output
    behind_collective: set = set()                             # nodes that (transitively) depend on a collective

    def ready_of(node: TaskNode, t: torch.Tensor, rows: int) -> Tuple[Optional[RowEvents], List[tuple]]:
        """Row-aligned events for tensor ``t`` if one dependency produced exactly this view; every other
        dependency becomes a whole-node wait."""
        aligned, extra = None, []
        for dep in node.depends_on:
            ent = produced.get(dep._node_id)
            if ent is None:
                continue
            dnode, ev = ent
            o = dnode.outputs[0]
            if (aligned is None and t is not None and o.data_ptr() == t.data_ptr() and o.numel() == t.numel()
                    and ev.rows == rows and o.numel() > 0):
                aligned = ev
            else:
                extra.append((ev.all_event[0], ev.all_event[1], ev.sys, False))
        return aligned, extra

    for node in graph._schedule.order if graph._schedule is not None else graph._nodes:
        t = node.task_type
        out = node.outputs[0] if node.outputs else None
        if out is None or out.numel() == 0:
            continue
        after_coll = any(d._node_id in behind_collective for d in node.depends_on)
        if dist and (t in _COLL or after_coll):
            behind_collective.add(node._node_id)
        if t in (TaskType.LINEAR, TaskType.MATMUL):
            x2 = _flat2d(node.inputs[0])
            w = node.inputs[1]
            aligned, extra = ready_of(node, node.inputs[0], x2.shape[0])
            act = node.attrs.get("activation")
            bias = node.inputs[2] if node.attrs.get("has_bias") else None
            out2 = out.view(-1, out.shape[-1])
            if node._node_id in fused_rs:
                # linear -> reduce_scatter: partial tiles leave through the GEMM epilogue; the product itself is
                # never written on this rank
                rs = fused_rs[node._node_id]
                gemm_ev, out_ev = gc.lower_linear_reduce_scatter(ctx, node, rs, aligned, extra, need_opening=not after_coll)
                behind_collective.add(rs._node_id)
                produced[node._node_id] = (node, gemm_ev)
                produced[rs._node_id] = (rs, out_ev)
                skip[rs._node_id] = True
                continue
            few_rows = (t == TaskType.LINEAR and bias is None and act in (None, "none", "swiglu") and x2.shape[0] <= BM
                        and w.shape[0] % 256 == 0 and x2.shape[1] % BK == 0 and w.shape[0] * w.shape[1] >= (1 << 22))
            if few_rows:
                # decode-shaped linear: a weight stream, cut along K over every SM (csrc/splitk_tasks.cuh)
                ev = b.gemm_splitk(x2, w, out2, epilogue=act if act == "swiglu" else None, a_ready=aligned, extra_waits=extra)
            else:
                order = None
                if dist and aligned is not None and aligned.sys and x2.shape[0] % (heap.world * BM) == 0:
                    # rows that arrive from other ranks (an all-gathered input): own shard first, then in arrival order
                    from ..parallel import fused as _fused
                    src = next((d for d in node.depends_on if d.task_type == TaskType.ALLGATHER
                                and d.outputs[0].data_ptr() == node.inputs[0].data_ptr()), None)
                    if src is not None:
                        order = _fused.gathered_order(heap.rank, heap.world, x2.shape[0] // heap.world // BM, False)
                ev = b.gemm(x2, w, out2, trans_b=(t == TaskType.MATMUL), epilogue=act, bias=bias,
                            a_ready=aligned, extra_waits=extra, m_blocks=order)
            produced[node._node_id] = (node, ev)
        elif t in _ELT_TYPES:
            x = node.inputs[0]
            cols = x.shape[-1]
            rows = x.numel() // cols
            kw = {}
            in1 = node.inputs[1] if len(node.inputs) > 1 else None
            in2 = node.inputs[2] if len(node.inputs) > 2 else None
            if t in (TaskType.RMSNORM, TaskType.LAYERNORM):
                kw["f0"] = node.attrs["eps"]
            elif t == TaskType.SCALE:
                kw["f0"] = node.attrs["factor"]
            elif t == TaskType.ROPE:
                tokens, heads, hd = x.shape
                rows, cols = tokens * heads, hd
                kw.update(i0=heads, i1=0, ld_in=heads * hd, ld_out=heads * hd)
            aligned, extra = ready_of(node, x, rows)
            readies = [aligned]
            if t in (TaskType.ADD, TaskType.SILU_GATE) and in1 is not None:
                # second operand: look for its own row-aligned producer among the remaining dependencies
                for dep in node.depends_on:
                    ent = produced.get(dep._node_id)
                    if ent and ent[0].outputs[0].data_ptr() == in1.data_ptr() and ent[1].rows == rows and ent[1] is not aligned:
                        readies.append(ent[1])
                        extra = [e for e in extra if e[0] != ent[1].all_event[0]]
                        break
            ev = b.elementwise(int(t), x, out, in1=in1, in2=in2, rows=rows, cols=cols, in_ready=readies,
                               extra_waits=extra, **kw)
            produced[node._node_id] = (node, ev)
        elif dist and t in _COLL:
            if skip.get(node._node_id):
                continue
            x = node.inputs[0]
            rows = x.numel() // max(1, x.shape[-1] if x.dim() else 1)
            aligned, extra = ready_of(node, x, rows)
            fn = {TaskType.ALLGATHER: gc.lower_allgather, TaskType.REDUCE_SCATTER: gc.lower_reduce_scatter,
                  TaskType.ALLREDUCE: gc.lower_allreduce, TaskType.BROADCAST: gc.lower_broadcast,
                  TaskType.ALL_TO_ALL: gc.lower_all_to_all}[t]
            produced[node._node_id] = (node, fn(ctx, node, aligned, extra))
        elif t in (TaskType.ALL_TO_ALL, TaskType.ALLGATHER, TaskType.REDUCE_SCATTER):
            # world size 1: the collective degenerates to a copy
            x = node.inputs[0]
            cols = x.shape[-1] if x.dim() else 1
            rows = x.numel() // max(1, cols)
            aligned, extra = ready_of(node, x, rows)
            ev = b.elementwise(300, x, out, rows=rows, cols=cols, in_ready=[aligned], extra_waits=extra)
            produced[node._node_id] = (node, ev)
        elif t in (TaskType.ALLREDUCE, TaskType.BROADCAST, TaskType.NOP):
            # in place and a no-op at world size 1: consumers inherit the producers of the tensor
            aligned, extra = ready_of(node, node.inputs[0] if node.inputs else None, -1)
            if aligned is not None:      # another in-place node on the same tensor (its events carry rows = -1 too)
                extra = extra + [(aligned.all_event[0], aligned.all_event[1], aligned.sys, False)]
            waits = b.join(extra, 0)
            e = b.new_event()
            b.add_task(int(TaskType.NOP), b"", waits=waits, signals=[e])
            produced[node._node_id] = (node, RowEvents(rows=-1, block=BM, row_events=[], all_event=(e, 1)))
        else:
            raise NotImplementedError(f"no task form for {t.name}")
    if ctx is not None:
        ctx.finish()
    prog = b.build()
    if ctx is not None:
        prog.heap_buffers = ctx.heap_buffers
    return prog


def graph_comm_workers(graph, workers: int) -> int:
    """Communication workers of a multi-rank graph program: the REMOTE_SCHEDULER share of the graph's SM
    configuration (``graph.sm_config``, an ``SMConfig``) when the user set one, else ``config.sm_policy``
    ("auto": the SMManager's automatic split; "compute": none; a number: that many)."""
    from ..config import config
    from ..core.sm_manager import SMManager
    smc = getattr(graph, "sm_config", None)
    policy = str(config.sm_policy).lower()
    if smc is not None:
        n = SMManager(smc, device=graph.device).get_worker_config()["num_remote_schedulers"]
    elif policy.isdigit():
        n = int(policy)
    elif policy in ("compute", "none"):
        n = 0
    else:
        n = SMManager(device=graph.device).get_worker_config()["num_remote_schedulers"]
    return max(0, min(n, workers - 2))
