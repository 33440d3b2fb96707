"""``LearnedQuery``: the trainable ``[rank]`` vector a read is queried with.

Behaviour follows src/attnres/modules.py:22-38 of the reference: the parameter is created in
BF16 from N(0, init_std); calling the module returns the parameter as BF16 whatever dtype the
module was later cast to, so an FP32 master copy trains through a BF16 query and receives an
FP32 gradient.  Bad arguments raise the same exception types as the reference
(tests/test_info.py:27-38, tests/test_api.py of the reference).
"""
from __future__ import annotations

import math
from numbers import Integral

import torch


def _length(rank) -> int:
    """``rank`` as a positive int; integer-like objects (``__index__``) are accepted, bools and
    floats are not."""
    if isinstance(rank, bool) or not (isinstance(rank, Integral) or hasattr(rank, "__index__")):
        raise TypeError("rank must be an integer")
    try:
        length = rank.__index__()
    except TypeError as error:
        raise TypeError("rank must be an integer") from error
    if length <= 0:
        raise ValueError("rank must be positive")
    return length


def _spread(init_std) -> float:
    value = float(init_std)
    if math.isnan(value) or math.isinf(value) or value <= 0.0:
        raise ValueError("init_std must be finite and positive")
    return value


class LearnedQuery(torch.nn.Module):
    """Holds one query vector of ``rank`` entries and hands it out in BF16."""

    def __init__(self, rank: int, *, init_std: float = 0.02) -> None:
        super().__init__()
        length, spread = _length(rank), _spread(init_std)
        start = torch.empty(length, dtype=torch.bfloat16).normal_(mean=0.0, std=spread)
        self.query = torch.nn.Parameter(start)

    def forward(self) -> torch.Tensor:
        # ``.to`` is the identity for a BF16 parameter and a differentiable cast otherwise
        return self.query.to(torch.bfloat16)


__all__ = ["LearnedQuery"]
