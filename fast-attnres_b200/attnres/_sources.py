"""Argument validation shared by the packed and source-list entry points.

Same checks, exception types and order as the reference
(src/attnres/_sources.py:16-93 and src/attnres/api.py:9-27); nothing here
copies, stacks or makes a tensor contiguous.
"""
from __future__ import annotations

import math
from numbers import Real

import torch

DEFAULT_EPS = 2**-23
MAX_SOURCES = 129
MAX_WIDTH = 8192
_BF16 = torch.bfloat16


def check_scalar(value, name: str, *, positive: bool = False) -> None:
    """Real, finite (and optionally positive) Python scalars only; bool is refused."""
    if isinstance(value, bool) or not isinstance(value, Real):
        raise TypeError(f"{name} must be a real scalar")
    number = float(value)
    if not math.isfinite(number) or (positive and number <= 0.0):
        raise ValueError(f"{name} must be {'finite and positive' if positive else 'finite'}")


def check_packed(values: torch.Tensor, query, eps, scale) -> None:
    """Validation of a packed ``[S, ..., D]`` call (src/attnres/api.py:9-27)."""
    if not isinstance(query, torch.Tensor):
        raise TypeError("query must be a tensor")
    if values.ndim < 2 or query.ndim != 1:
        raise ValueError("expected values [S,...,D] and query [R]")
    if not 1 <= values.shape[0] <= MAX_SOURCES or not 1 <= values.shape[-1] <= MAX_WIDTH:
        raise ValueError(f"supported envelope is 1<=S<={MAX_SOURCES} and 1<=D<={MAX_WIDTH}")
    if any(size < 1 for size in values.shape) or not 1 <= query.numel() <= values.shape[-1]:
        raise ValueError("dimensions must be positive and 1<=R<=D")
    if values.dtype != _BF16:
        raise TypeError("values must use BF16 storage")
    if query.dtype != _BF16:
        raise TypeError("query must use BF16 storage")
    if query.device != values.device:
        raise TypeError("query must be on the values device")
    check_scalar(eps, "eps", positive=True)
    check_scalar(scale, "scale")
    if not values.is_cuda:
        raise RuntimeError("attnres requires CUDA tensors")


def check_sources(values, query, eps, scale) -> tuple[torch.Tensor, ...]:
    """Validation of a list/tuple call; returns the sources as a tuple, untouched
    (src/attnres/_sources.py:37-93)."""
    if not isinstance(query, torch.Tensor):
        raise TypeError("query must be a tensor")
    if query.ndim != 1:
        raise ValueError("query must have 1 dimensions")
    if any(int(size) < 1 for size in query.shape):
        raise ValueError("query dimensions must be positive")
    if query.dtype != _BF16:
        raise TypeError("query must use BF16 storage")
    if not isinstance(values, (list, tuple)):
        raise TypeError("values must be a tensor or a list/tuple of tensors")
    sources = tuple(values)
    if not 1 <= len(sources) <= MAX_SOURCES:
        raise ValueError(f"supported source envelope is 1<=S<={MAX_SOURCES}")
    if any(not isinstance(source, torch.Tensor) for source in sources):
        raise TypeError("values must contain only tensors")
    first = sources[0]
    if first.ndim < 1:
        raise ValueError("each source must have shape [...,D]")
    if any(int(size) < 1 for size in first.shape):
        raise ValueError("source dimensions must be positive")
    width = int(first.shape[-1])
    if not 1 <= width <= MAX_WIDTH:
        raise ValueError(f"supported value envelope is 1<=D<={MAX_WIDTH}")
    if first.dtype != _BF16:
        raise TypeError("values must use BF16 storage")
    if query.device != first.device:
        raise TypeError("query must be on the values device")
    for index, source in enumerate(sources):
        if source.ndim < 1:
            raise ValueError(f"source {index} must have shape [...,D]")
        if tuple(source.shape) != tuple(first.shape):
            raise ValueError("all source tensors must have the same logical shape")
        if source.dtype != first.dtype or source.device != first.device:
            raise TypeError("all source tensors must match the first source dtype/device")
    if not 1 <= int(query.shape[-1]) <= width:
        raise ValueError("query rank must satisfy 1<=R<=D")
    check_scalar(eps, "eps", positive=True)
    check_scalar(scale, "scale")
    return sources


def row_layout(tensor: torch.Tensor) -> tuple[torch.Tensor, int, int]:
    """Describe ``tensor [..., D]`` as rows: ``(tensor, row_stride, feature_stride)``.

    The leading axes are flattened to one row index when their strides allow it
    (size-1 axes never constrain the layout); otherwise the tensor is made
    contiguous first.  The reference has the same rule
    (src/attnres/_kernels/fla_full_sources.py:164-214); only a source whose
    batch axes are not affine is ever copied.
    """
    row_stride = _affine_row_stride(tensor)
    if row_stride is None:
        tensor = tensor.contiguous()
        row_stride = _affine_row_stride(tensor)
    return tensor, int(row_stride), int(tensor.stride(-1))


def _affine_row_stride(tensor: torch.Tensor):
    stride_of_row = None
    rows_inside = 1
    for size, stride in zip(reversed(tensor.shape[:-1]), reversed(tensor.stride()[:-1])):
        size, stride = int(size), int(stride)
        if size == 1:
            continue
        if stride_of_row is None:
            stride_of_row = stride
        elif stride != rows_inside * stride_of_row:
            return None
        rows_inside *= size
    return 0 if stride_of_row is None else stride_of_row


__all__ = ["DEFAULT_EPS", "MAX_SOURCES", "MAX_WIDTH", "check_packed", "check_scalar",
           "check_sources", "row_layout"]
