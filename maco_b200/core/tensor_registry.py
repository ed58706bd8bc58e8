"""Name -> tensor registry (reference: maco/core/tensor_registry.py:12-161)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch


@dataclass
class TensorInfo:
    name: str
    tensor: torch.Tensor
    shape: Tuple[int, ...]
    dtype: torch.dtype
    is_weight: bool = False
    is_input: bool = False
    is_output: bool = False
    device_ptr: int = 0


class TensorRegistry:
    def __init__(self):
        self._tensors: Dict[str, TensorInfo] = {}

    def register(self, tensor: torch.Tensor, name: str, is_weight: bool = False, is_input: bool = False,
                 is_output: bool = False) -> TensorInfo:
        if name in self._tensors:
            raise ValueError(f"tensor {name!r} is already registered")
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"expected a tensor for {name!r}, got {type(tensor).__name__}")
        info = TensorInfo(name, tensor, tuple(tensor.shape), tensor.dtype, is_weight, is_input, is_output,
                          tensor.data_ptr() if tensor.numel() else 0)
        self._tensors[name] = info
        return info

    def register_input(self, tensor, name): return self.register(tensor, name, is_input=True)
    def register_weight(self, tensor, name): return self.register(tensor, name, is_weight=True)

    def register_output(self, tensor_or_shape, name: str, dtype: torch.dtype = torch.float32, device=None) -> TensorInfo:
        if isinstance(tensor_or_shape, torch.Tensor):
            t = tensor_or_shape
        else:
            t = torch.empty(tuple(tensor_or_shape), dtype=dtype, device=device)
        return self.register(t, name, is_output=True)

    def get(self, name: str) -> Optional[TensorInfo]:
        return self._tensors.get(name)

    def get_tensor(self, name: str) -> Optional[torch.Tensor]:
        info = self._tensors.get(name)
        return info.tensor if info else None

    @property
    def inputs(self): return {k: v for k, v in self._tensors.items() if v.is_input}
    @property
    def outputs(self): return {k: v for k, v in self._tensors.items() if v.is_output}
    @property
    def weights(self): return {k: v for k, v in self._tensors.items() if v.is_weight}

    def get_all_pointers(self) -> Dict[str, int]:
        return {k: v.device_ptr for k, v in self._tensors.items()}

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {k: v.tensor.detach().clone() for k, v in self.weights.items()}

    def clear(self) -> None:
        self._tensors.clear()

    def __len__(self) -> int:
        return len(self._tensors)

    def __contains__(self, name: str) -> bool:
        return name in self._tensors
