"""Argument checks for the graph-building calls.

Mirrors the helper set of the reference's maco/task_graph/validation.py:19-241. One deliberate
difference: the reference hard-requires CUDA tensors (``require_cuda=True``, validation.py:27,58-59)
even though its TaskGraph falls back to a CPU device; here the rule is "the tensor's device type
must equal the graph's device type", so a CPU graph accepts CPU tensors and a CUDA graph still
raises DeviceError for them.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .exceptions import (
    DeviceError,
    DimensionError,
    DTypeMismatchError,
    NullInputError,
    ShapeMismatchError,
    ValidationError,
)


def validate_tensor(
    tensor,
    name: str,
    method: str,
    *,
    ndim: Optional[int] = None,
    min_ndim: Optional[int] = None,
    max_ndim: Optional[int] = None,
    require_cuda: bool = False,
    device: Optional[torch.device] = None,
) -> None:
    if tensor is None:
        raise NullInputError(name, method)
    if not isinstance(tensor, torch.Tensor):
        raise ValidationError(
            f"'{name}' must be a torch.Tensor in {method}(), got {type(tensor).__name__}\n"
            f"Hint: wrap the data with torch.as_tensor(...)"
        )
    if require_cuda and not tensor.is_cuda:
        raise DeviceError(name, str(tensor.device), "cuda")
    if device is not None:
        want = torch.device(device)
        if tensor.device.type != want.type:
            raise DeviceError(name, str(tensor.device), str(want.type))
        if want.type == "cuda" and want.index is not None and tensor.device.index != want.index:
            raise DeviceError(name, str(tensor.device), str(want))
    if ndim is not None and tensor.dim() != ndim:
        raise DimensionError(name, ndim, tensor.dim())
    if min_ndim is not None and tensor.dim() < min_ndim:
        raise DimensionError(name, f">={min_ndim}", tensor.dim())
    if max_ndim is not None and tensor.dim() > max_ndim:
        raise DimensionError(name, f"<={max_ndim}", tensor.dim())


def validate_linear_shapes(input: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    in_features = input.shape[-1]
    if weight.dim() != 2:
        raise DimensionError("weight", 2, weight.dim())
    if weight.shape[1] != in_features:
        raise ShapeMismatchError(
            "linear",
            f"input.shape[-1]={in_features} != weight.shape[1]={weight.shape[1]} "
            f"(input {tuple(input.shape)}, weight {tuple(weight.shape)})",
            "weight must be [out_features, in_features] with in_features equal to the input's last dimension",
        )
    if bias is not None:
        if bias.dim() != 1 or bias.shape[0] != weight.shape[0]:
            raise ShapeMismatchError(
                "linear",
                f"bias shape {tuple(bias.shape)} does not match out_features={weight.shape[0]}",
                "bias must be a vector of length weight.shape[0]",
            )


def validate_matmul_shapes(a: torch.Tensor, b: torch.Tensor) -> None:
    if a.shape[-1] != b.shape[-2 if b.dim() >= 2 else 0]:
        raise ShapeMismatchError(
            "matmul",
            f"a.shape[-1]={a.shape[-1]} != b.shape[-2]={b.shape[-2 if b.dim() >= 2 else 0]} "
            f"(a {tuple(a.shape)}, b {tuple(b.shape)})",
            "the inner dimensions must agree: a is [..., M, K], b is [K, N]",
        )


def validate_dtype_match(t1: torch.Tensor, name1: str, t2: torch.Tensor, name2: str) -> None:
    if t1.dtype != t2.dtype:
        raise DTypeMismatchError(name1, t1.dtype, name2, t2.dtype)


def validate_same_device(tensors: Sequence[torch.Tensor], names: Sequence[str]) -> None:
    if not tensors:
        return
    first = tensors[0].device
    for t, n in zip(tensors[1:], names[1:]):
        if t.device != first:
            raise DeviceError(n, str(t.device), str(first))


def infer_device(*tensors) -> Optional[torch.device]:
    for t in tensors:
        if isinstance(t, torch.Tensor):
            return t.device
    return None


def infer_dtype(*tensors) -> Optional[torch.dtype]:
    for t in tensors:
        if isinstance(t, torch.Tensor):
            return t.dtype
    return None
