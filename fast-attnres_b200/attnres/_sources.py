"""Argument checks of the packed and the source-list entry points, and the row layout of a
source.

A call is refused with the exception TYPE the reference raises for the same mistake, and when
several things are wrong the same one is reported first (src/attnres/api.py:9-27 for a packed
tensor, src/attnres/_sources.py:16-93 for a list): wrong container or element types and wrong
dtypes or devices are ``TypeError``; ranks, extents, the S <= 129 / D <= 8192 / R <= D envelope
and non-finite scalars are ``ValueError``; CPU tensors are ``RuntimeError`` and are reported
last.  Each entry point is an ordered table of (condition that must hold, exception, message);
the first condition that fails decides.  Nothing here copies, stacks or re-lays-out a tensor.
"""
from __future__ import annotations

import math
from numbers import Real

import torch

DEFAULT_EPS = 2**-23
MAX_SOURCES = 129
MAX_WIDTH = 8192
_BF16 = torch.bfloat16


def _first_failure(rules) -> None:
    """Raise for the first rule whose condition does not hold; conditions are evaluated
    lazily and in order, so a later one may rely on the earlier ones."""
    for holds, kind, message in rules:
        if not holds():
            raise kind(message)


def check_scalar(value, name: str, *, positive: bool = False) -> None:
    """``eps`` / ``scale``: a real Python number (not a bool, string or tensor), finite, and
    for ``positive=True`` greater than zero."""
    wanted = "finite and positive" if positive else "finite"
    _first_failure((
        (lambda: isinstance(value, Real) and not isinstance(value, bool), TypeError,
         f"{name} must be a real scalar"),
        (lambda: math.isfinite(float(value)), ValueError, f"{name} must be {wanted}"),
        (lambda: not positive or float(value) > 0.0, ValueError, f"{name} must be {wanted}"),
    ))


def check_packed(values: torch.Tensor, query, eps, scale) -> None:
    """A packed call: ``values`` is ``[S, ..., D]``, ``query`` is ``[R]``."""
    envelope = f"supported envelope is 1<=S<={MAX_SOURCES} and 1<=D<={MAX_WIDTH}"
    _first_failure((
        (lambda: isinstance(query, torch.Tensor), TypeError, "query must be a tensor"),
        (lambda: values.ndim >= 2 and query.ndim == 1, ValueError,
         "expected values [S,...,D] and query [R]"),
        (lambda: 1 <= values.shape[0] <= MAX_SOURCES and 1 <= values.shape[-1] <= MAX_WIDTH,
         ValueError, envelope),
        (lambda: min(values.shape) >= 1 and 1 <= query.numel() <= values.shape[-1], ValueError,
         "dimensions must be positive and 1<=R<=D"),
        (lambda: values.dtype == _BF16, TypeError, "values must use BF16 storage"),
        (lambda: query.dtype == _BF16, TypeError, "query must use BF16 storage"),
        (lambda: query.device == values.device, TypeError, "query must be on the values device"),
    ))
    check_scalar(eps, "eps", positive=True)
    check_scalar(scale, "scale")
    if not values.is_cuda:
        raise RuntimeError("attnres requires CUDA tensors")


def check_sources(values, query, eps, scale) -> tuple[torch.Tensor, ...]:
    """A list/tuple call: S tensors ``[..., D]`` of one shape, dtype and device.  Returns the
    sources as a tuple of the very same tensor objects."""
    _first_failure((
        (lambda: isinstance(query, torch.Tensor), TypeError, "query must be a tensor"),
        (lambda: query.ndim == 1, ValueError, "query must have 1 dimensions"),
        (lambda: query.numel() >= 1, ValueError, "query dimensions must be positive"),
        (lambda: query.dtype == _BF16, TypeError, "query must use BF16 storage"),
        (lambda: isinstance(values, (list, tuple)), TypeError,
         "values must be a tensor or a list/tuple of tensors"),
        (lambda: 1 <= len(values) <= MAX_SOURCES, ValueError,
         f"supported source envelope is 1<=S<={MAX_SOURCES}"),
        (lambda: all(isinstance(item, torch.Tensor) for item in values), TypeError,
         "values must contain only tensors"),
    ))
    sources = tuple(values)
    head = sources[0]
    _first_failure((
        (lambda: head.ndim >= 1, ValueError, "each source must have shape [...,D]"),
        (lambda: min(head.shape) >= 1, ValueError, "source dimensions must be positive"),
        (lambda: head.shape[-1] <= MAX_WIDTH, ValueError,
         f"supported value envelope is 1<=D<={MAX_WIDTH}"),
        (lambda: head.dtype == _BF16, TypeError, "values must use BF16 storage"),
        (lambda: query.device == head.device, TypeError, "query must be on the values device"),
    ))
    for position, item in enumerate(sources):
        _first_failure((
            (lambda: item.ndim >= 1, ValueError, f"source {position} must have shape [...,D]"),
            (lambda: item.shape == head.shape, ValueError,
             "all source tensors must have the same logical shape"),
            (lambda: item.dtype == head.dtype and item.device == head.device, TypeError,
             "all source tensors must match the first source dtype/device"),
        ))
    if query.numel() > head.shape[-1]:
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
