"""Helpers around the core: the CPU model of the scheduling protocol and the input prefetcher."""
from .prefetch import InputPrefetcher

__all__ = ["InputPrefetcher"]
