"""Core layer: SM roles, contexts, tensor registry (reference: maco/core/__init__.py:1-14)."""
from .context import Context, PersistentContext
from .sm_demo import run_sm_scheduling_demo
from .sm_manager import Role, SMAssignment, SMConfig, SMManager, auto_config
from .tensor_registry import TensorInfo, TensorRegistry

__all__ = ["SMConfig", "SMManager", "SMAssignment", "Role", "auto_config", "Context", "PersistentContext",
           "TensorRegistry", "TensorInfo", "run_sm_scheduling_demo"]
