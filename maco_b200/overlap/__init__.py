"""Compute / communication overlap on two streams (reference: maco/overlap/__init__.py)."""
from .manager import OverlapManager, OverlapRegion, OverlapTask

__all__ = ["OverlapManager", "OverlapRegion", "OverlapTask"]
