"""Process-group ownership: rank, world size, device, the communication stream, heartbeats.

Surface of the reference's ProcessGroupManager (maco/comm/process_group.py:13-199): a singleton
that adopts an already-initialised torch.distributed group or creates one from the environment
(RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT). Added here: a side gloo group for
host-side exchanges (symmetric-heap handles), and store-based heartbeats so that ranks learn on
the host, before their next launch, that a peer has stopped (the reference has no failure path).
"""
from __future__ import annotations

import datetime
import os
import time
from typing import List, Optional

import torch
import torch.distributed as dist


class ProcessGroupManager:
    _instance: Optional["ProcessGroupManager"] = None

    def __new__(cls):
        if cls._instance is None:
            inst = super().__new__(cls)
            inst._initialized = False
            inst._world_size = 1
            inst._rank = 0
            inst._local_rank = 0
            inst._device = None
            inst._comm_stream = None
            inst._owns_group = False
            inst._backend = None
            inst._host_group = None
            inst._store = None
            inst._hb_prefix = "maco_hb"
            cls._instance = inst
        return cls._instance

    # ------------------------------------------------------------------ init / destroy
    def init_process_group(self, backend: str = "nccl", init_method: Optional[str] = None,
                           world_size: Optional[int] = None, rank: Optional[int] = None,
                           timeout_s: Optional[float] = None) -> "ProcessGroupManager":
        if self._initialized:
            return self
        if dist.is_available() and dist.is_initialized():
            self._sync_from_dist()
        else:
            env = os.environ
            world = int(world_size if world_size is not None else env.get("WORLD_SIZE", 1))
            rk = int(rank if rank is not None else env.get("RANK", 0))
            self._local_rank = int(env.get("LOCAL_RANK", rk))
            if backend == "nccl" and not torch.cuda.is_available():
                backend = "gloo"
            if world > 1:
                kwargs = {}
                if timeout_s is not None:
                    kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
                if backend == "nccl":
                    torch.cuda.set_device(self._local_rank % max(1, torch.cuda.device_count()))
                    kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
                dist.init_process_group(backend=backend, init_method=init_method or "env://",
                                        world_size=world, rank=rk, **kwargs)
                self._owns_group = True
            self._world_size, self._rank, self._backend = world, rk, backend
        self._setup_device()
        self._initialized = True
        return self

    def _sync_from_dist(self) -> None:
        self._world_size = dist.get_world_size()
        self._rank = dist.get_rank()
        self._local_rank = int(os.environ.get("LOCAL_RANK", self._rank))
        self._backend = dist.get_backend()

    def _setup_device(self) -> None:
        if torch.cuda.is_available() and self._backend != "gloo":
            idx = self._local_rank % torch.cuda.device_count()
            torch.cuda.set_device(idx)
            self._device = torch.device("cuda", idx)
            self._comm_stream = torch.cuda.Stream(device=self._device)
        else:
            self._device = torch.device("cpu")
            self._comm_stream = None

    def destroy(self) -> None:
        if self._owns_group and dist.is_initialized():
            dist.destroy_process_group()
        ProcessGroupManager._instance = None

    # ------------------------------------------------------------------ properties
    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def local_rank(self) -> int:
        return self._local_rank

    @property
    def device(self) -> torch.device:
        return self._device if self._device is not None else torch.device("cpu")

    @property
    def comm_stream(self):
        return self._comm_stream

    @property
    def backend(self) -> Optional[str]:
        return self._backend

    @property
    def is_main_process(self) -> bool:
        return self._rank == 0

    @property
    def is_initialized(self) -> bool:
        return self._initialized

    def barrier(self) -> None:
        if self._world_size > 1 and dist.is_initialized():
            dist.barrier()

    # ------------------------------------------------------------------ host-side exchange
    def host_group(self):
        """A gloo group over the same ranks, for exchanging Python objects and handles."""
        if self._world_size <= 1 or not dist.is_initialized():
            return None
        if self._backend == "gloo":
            return dist.group.WORLD
        if self._host_group is None:
            self._host_group = dist.new_group(backend="gloo")
        return self._host_group

    def all_gather_object(self, obj) -> List:
        if self._world_size <= 1 or not dist.is_initialized():
            return [obj]
        out = [None] * self._world_size
        dist.all_gather_object(out, obj, group=self.host_group())
        return out

    # ------------------------------------------------------------------ heartbeats (failure detection)
    def _get_store(self):
        if self._store is None and dist.is_initialized():
            self._store = dist.distributed_c10d._get_default_store()
        return self._store

    def heartbeat(self, step: int) -> None:
        """Publishes "rank r reached step" in the rendezvous store."""
        store = self._get_store()
        self._last_step = int(step)
        if store is not None:
            store.set(f"{self._hb_prefix}/{self._rank}", f"{step}:{time.time():.3f}")

    def announce_exit(self) -> None:
        """Publishes that this rank leaves after the last step it reported (call between steps)."""
        store = self._get_store()
        if store is not None:
            store.set(f"{self._hb_prefix}/{self._rank}", f"exit:{getattr(self, '_last_step', -1)}")

    def check_peers(self, step: int, timeout_s: float = 5.0, poll_s: float = 0.01) -> List[int]:
        """Returns the ranks that have NOT reached ``step`` within ``timeout_s`` (or announced exit)."""
        store = self._get_store()
        if store is None:
            return []
        lost: List[int] = []
        deadline = time.time() + timeout_s
        for r in range(self._world_size):
            if r == self._rank:
                continue
            key = f"{self._hb_prefix}/{r}"
            ok = False
            while True:
                try:
                    if store.check([key]):
                        val = store.get(key).decode()
                        head, tail = val.split(":")[0], val.split(":")[1]
                        if head == "exit":
                            ok = int(tail) >= step      # it had reached this step before it left
                            break
                        if int(head) >= step:
                            ok = True
                            break
                except Exception:
                    pass
                if time.time() >= deadline:
                    break
                time.sleep(poll_s)
            if not ok:
                lost.append(r)
        return lost


def ensure_peers(step: int, timeout_s: float = 5.0) -> None:
    """Publishes this rank's heartbeat for ``step`` and raises PeerLostError when a peer has not reached
    it (or has announced that it left). Call between steps, before launching anything that waits on peers."""
    from ..task_graph.exceptions import PeerLostError
    m = ProcessGroupManager()
    m.heartbeat(step)
    lost = m.check_peers(step, timeout_s=timeout_s)
    if lost:
        raise PeerLostError(lost[0], f"ranks {lost} did not reach step {step}")


def _mgr() -> ProcessGroupManager:
    return ProcessGroupManager()


def get_world_size() -> int:
    m = ProcessGroupManager._instance
    if m is not None and m.is_initialized:
        return m.world_size
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size()
    return 1


def get_rank() -> int:
    m = ProcessGroupManager._instance
    if m is not None and m.is_initialized:
        return m.rank
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank()
    return 0


def get_local_rank() -> int:
    m = ProcessGroupManager._instance
    if m is not None and m.is_initialized:
        return m.local_rank
    return int(os.environ.get("LOCAL_RANK", 0))


def is_initialized() -> bool:
    m = ProcessGroupManager._instance
    return bool(m is not None and m.is_initialized) or (dist.is_available() and dist.is_initialized())


def barrier() -> None:
    if get_world_size() > 1 and dist.is_initialized():
        dist.barrier()
