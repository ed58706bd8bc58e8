"""Helpers around the core: the CPU model of the scheduling protocol, the input prefetcher and the
pipelined end-to-end step loop."""
from .prefetch import InputPrefetcher, StepPipeline

__all__ = ["InputPrefetcher", "StepPipeline"]
