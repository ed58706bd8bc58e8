"""Helpers around the core: the CPU model of the scheduling protocol, the input prefetcher, the
pipelined end-to-end step loop and the host-side placement next to the GPU."""
from .numa import bind_host_to_gpu, local_cpus
from .prefetch import InputPrefetcher, StepPipeline

__all__ = ["InputPrefetcher", "StepPipeline", "bind_host_to_gpu", "local_cpus"]
