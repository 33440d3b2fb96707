"""Trainable query parameter for the AttnRes read.

Mirrors src/attnres/modules.py:22-38: a BF16 ``[rank]`` parameter drawn from
N(0, init_std); ``forward()`` always hands the operator a BF16 tensor, so a
module cast to FP32 still trains (FP32 parameter, BF16 query, FP32 gradient).
"""
from __future__ import annotations

import math
import operator

import torch
from torch import nn


def _as_index(value, name: str) -> int:
    if isinstance(value, bool):
        raise TypeError(f"{name} must be an integer")
    try:
        return operator.index(value)
    except TypeError as error:
        raise TypeError(f"{name} must be an integer") from error


class LearnedQuery(nn.Module):
    """A static trainable query vector of length ``rank``."""

    def __init__(self, rank: int, *, init_std: float = 0.02) -> None:
        super().__init__()
        rank = _as_index(rank, "rank")
        init_std = float(init_std)
        if rank < 1:
            raise ValueError("rank must be positive")
        if not math.isfinite(init_std) or init_std <= 0:
            raise ValueError("init_std must be finite and positive")
        self.query = nn.Parameter(torch.empty(rank, dtype=torch.bfloat16))
        nn.init.normal_(self.query, mean=0.0, std=init_std)

    def forward(self) -> torch.Tensor:
        return self.query.to(dtype=torch.bfloat16)


__all__ = ["LearnedQuery"]
