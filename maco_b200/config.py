"""Global configuration object.

Same fields and methods as the reference's MacoConfig (maco/config.py:9-61), where nothing reads
them. Here they are live: ``backend`` selects the collective implementation ("peer" = in-kernel
collectives over NVLink peer memory, "nccl"/"gloo" = torch.distributed), ``comm_buffer_size`` sizes
the symmetric heap, ``heap_mode`` how it is shared (with or without an NVSwitch multicast binding), ``profile`` turns the device trace ring on, ``runtime`` picks the TaskGraph
executor. ``MACO_*`` environment variables override the defaults.
"""
from __future__ import annotations

import os
from dataclasses import asdict, dataclass, fields
from typing import Any, Dict


def _parse_size(text) -> int:
    if isinstance(text, int):
        return text
    s = str(text).strip().upper()
    for suffix, mult in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10), ("B", 1)):
        if s.endswith(suffix):
            return int(float(s[: -len(suffix)]) * mult)
    return int(s)


@dataclass
class MacoConfig:
    backend: str = "peer"                 # "peer" | "nccl" | "gloo"
    sm_policy: str = "auto"               # communication workers of multi-rank graphs: "auto" (SMManager) | "compute" (none) | "<n>"
    overlap_strategy: str = "auto"        # "auto" | "wave" | "pipeline" | "none": stream-level overlap of comm nodes / OverlapRuntime default
    comm_buffer_size: str = "256MB"       # symmetric heap size per rank
    heap_mode: str = "auto"               # "auto" | "nvls" (multicast-bound) | "vmm" (shared descriptors) | "ipc" (cudaMalloc + IPC)
    use_pinned_memory: bool = True        # host staging of the input feed / result read-back goes through pinned memory
    runtime: str = "auto"                 # "auto" | "persistent" | "stream" | "reference"
    allow_tf32: bool = False              # fp32 GEMMs on the tensor cores as TF32 (10-bit mantissa) instead of CUDA-core fp32
    wait_budget_ms: float = 2000.0        # every device-side wait gives up after this long
    debug: bool = False                   # kernels re-check every task descriptor before running it (BAD_TASK on failure)
    profile: bool = False
    verbose: bool = False

    def __post_init__(self):
        env = os.environ
        self.backend = env.get("MACO_BACKEND", self.backend)
        self.runtime = env.get("MACO_RUNTIME", self.runtime)
        self.comm_buffer_size = env.get("MACO_COMM_BUFFER_SIZE", self.comm_buffer_size)
        self.heap_mode = env.get("MACO_HEAP", self.heap_mode)
        if "MACO_WAIT_BUDGET_MS" in env:
            self.wait_budget_ms = float(env["MACO_WAIT_BUDGET_MS"])
        for flag in ("debug", "profile", "verbose", "allow_tf32"):
            key = f"MACO_{flag.upper()}"
            if key in env:
                setattr(self, flag, env[key] not in ("0", "", "false", "False"))
        if env.get("MACO_TRACE", "0") not in ("0", ""):
            self.profile = True

    def set(self, **kwargs) -> "MacoConfig":
        known = {f.name for f in fields(self)}
        for k, v in kwargs.items():
            if k not in known:
                raise ValueError(f"Unknown config option: {k} (known: {sorted(known)})")
            setattr(self, k, v)
        return self

    def get(self, key: str, default: Any = None) -> Any:
        return getattr(self, key, default)

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @property
    def comm_buffer_bytes(self) -> int:
        return _parse_size(self.comm_buffer_size)


config = MacoConfig()
