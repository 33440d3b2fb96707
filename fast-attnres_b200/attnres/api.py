"""Public functional entry point (same contract as src/attnres/api.py:30-62)."""
from __future__ import annotations

import torch
from torch import Tensor

from ._sources import DEFAULT_EPS, check_packed, check_sources


def attnres(
    values: Tensor | list[Tensor] | tuple[Tensor, ...],
    query: Tensor,
    *,
    eps: float = DEFAULT_EPS,
    scale: float = 1.0,
) -> Tensor:
    """Mix source values with a static query over implicit tail keys.

    ``values`` is a packed ``[S, ..., D]`` tensor or an ordered list/tuple of
    ``S`` tensors ``[..., D]``; ``query`` is ``[R]`` with ``1 <= R <= D``.  The
    key of a source is its final ``R`` features, RMS-normalised; the softmax runs
    over the source axis independently at every position and the result keeps
    the full width ``D``.  Inputs and outputs are CUDA BF16 tensors; reductions
    are FP32.  First-order gradients flow to every source and to the query.
    """
    if isinstance(values, torch.Tensor):
        check_packed(values, query, eps, scale)
        from ._ops import packed_read  # the CUDA library loads on first GPU use only

        return packed_read(values, query, eps, scale)

    sources = check_sources(values, query, eps, scale)
    if not sources[0].is_cuda:
        raise RuntimeError("attnres requires CUDA tensors")
    from ._ops import sources_read

    return sources_read(sources, query, eps, scale)


__all__ = ["attnres"]
