"""SM role assignment: which SMs compute, which schedule, which serve communication.

API of the reference's maco/core/sm_manager.py:14-227 (``Role``, ``SMAssignment``, ``SMConfig``,
``SMManager``, ``auto_config``). In the reference the numbers are stored and never enforced. Here a multi-rank
``TaskGraph`` lowered to the persistent kernel takes its number of communication workers from
``SMManager.get_worker_config()["num_remote_schedulers"]`` (the graph's ``sm_config`` attribute when set, else the
automatic split, see ``ops.megakernel.graph_comm_workers``), and ``PersistentContext`` its worker count; the
hand-assembled model programs (``maco_b200.models``) pass their own measured counts.

B200 sizing (148 SMs): the scheduler needs one CTA; NVLink 5 copies saturate with roughly 8-16
CTAs issuing 16-byte peer stores, so the communication share is far smaller than the
reference's fixed 25 %.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional, Tuple

import torch

B200_SM_COUNT = 148


class Role(Enum):
    COMPUTE = "compute"
    LOCAL_SCHEDULER = "local_scheduler"      # the scheduler CTA(s) of the persistent kernel
    REMOTE_SCHEDULER = "remote_scheduler"    # CTAs that run communication tasks (peer copies / reductions)


@dataclass
class SMAssignment:
    sm_range: Tuple[int, int]                # [start, end)
    role: Role
    task_types: List[str] = field(default_factory=list)


def _detect_sms(device=None) -> int:
    if torch.cuda.is_available():
        return torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count
    return B200_SM_COUNT


@dataclass
class SMConfig:
    total_sms: int = 0
    assignments: List[SMAssignment] = field(default_factory=list)

    def __post_init__(self):
        if self.total_sms <= 0:
            self.total_sms = _detect_sms()

    def assign_role(self, sm_range: Tuple[int, int], role: Role, task_types: Optional[List[str]] = None) -> "SMConfig":
        lo, hi = int(sm_range[0]), int(sm_range[1])
        if lo < 0 or hi <= lo:
            raise ValueError(f"SM range {sm_range} is empty or negative")
        if hi > self.total_sms:
            raise ValueError(f"SM range {sm_range} exceeds total SMs ({self.total_sms})")
        for a in self.assignments:
            if lo < a.sm_range[1] and a.sm_range[0] < hi:
                raise ValueError(f"SM range {sm_range} overlaps with existing assignment {a.sm_range}")
        self.assignments.append(SMAssignment((lo, hi), role, list(task_types or [])))
        return self

    def _count(self, role: Role) -> int:
        return sum(a.sm_range[1] - a.sm_range[0] for a in self.assignments if a.role == role)

    @property
    def compute_sms(self) -> int:
        return self._count(Role.COMPUTE)

    @property
    def local_scheduler_sms(self) -> int:
        return self._count(Role.LOCAL_SCHEDULER)

    @property
    def remote_scheduler_sms(self) -> int:
        return self._count(Role.REMOTE_SCHEDULER)

    def validate(self) -> bool:
        if self.compute_sms <= 0:
            raise ValueError("SM configuration has no COMPUTE SMs")
        if self.compute_sms + self.local_scheduler_sms + self.remote_scheduler_sms > self.total_sms:
            raise ValueError("SM configuration assigns more SMs than the device has")
        return True

    def to_dict(self) -> dict:
        return {
            "total_sms": self.total_sms,
            "compute_sms": self.compute_sms,
            "local_scheduler_sms": self.local_scheduler_sms,
            "remote_scheduler_sms": self.remote_scheduler_sms,
            "assignments": [{"sm_range": a.sm_range, "role": a.role.value, "task_types": a.task_types}
                            for a in self.assignments],
        }


def _split(total: int, compute_ratio: float, local_ratio: float) -> SMConfig:
    cfg = SMConfig(total_sms=total)
    compute_end = max(1, min(total, int(total * compute_ratio)))
    local_end = max(compute_end, min(total, int(total * (compute_ratio + local_ratio))))
    cfg.assign_role((0, compute_end), Role.COMPUTE)
    if local_end > compute_end:
        cfg.assign_role((compute_end, local_end), Role.LOCAL_SCHEDULER)
    if total > local_end:
        cfg.assign_role((local_end, total), Role.REMOTE_SCHEDULER)
    return cfg


class SMManager:
    def __init__(self, config: Optional[SMConfig] = None, device=None):
        self.device = device
        self.config = config or self._auto_config()
        self._compiled = False

    def _auto_config(self) -> SMConfig:
        total = _detect_sms(self.device)
        cfg = SMConfig(total_sms=total)
        sched = 1
        comm = 8 if total >= 64 else max(0, total // 8)
        compute = total - sched - comm
        cfg.assign_role((0, compute), Role.COMPUTE)
        cfg.assign_role((compute, compute + sched), Role.LOCAL_SCHEDULER)
        if comm:
            cfg.assign_role((compute + sched, total), Role.REMOTE_SCHEDULER)
        return cfg

    def compile(self) -> "SMManager":
        self.config.validate()
        self._compiled = True
        return self

    def get_worker_config(self) -> dict:
        if not self._compiled:
            self.compile()
        return {
            "num_workers": self.config.compute_sms,
            "num_local_schedulers": self.config.local_scheduler_sms,
            "num_remote_schedulers": self.config.remote_scheduler_sms,
        }


_INTENSITY = {
    ("high", "low"): (0.90, 0.08), ("high", "medium"): (0.80, 0.15), ("high", "high"): (0.70, 0.20),
    ("medium", "low"): (0.85, 0.12), ("medium", "medium"): (0.75, 0.18), ("medium", "high"): (0.65, 0.23),
    ("low", "low"): (0.80, 0.15), ("low", "medium"): (0.70, 0.20), ("low", "high"): (0.60, 0.25),
}


def auto_config(compute_intensity: str = "high", comm_intensity: str = "medium", gpu_arch: str = "auto",
                total_sms: Optional[int] = None) -> SMConfig:
    """Role split from a coarse workload description (same 3x3 ratio table as the reference)."""
    total = total_sms if total_sms is not None else _detect_sms()
    c, l = _INTENSITY.get((compute_intensity, comm_intensity), (0.75, 0.18))
    return _split(total, c, l)
