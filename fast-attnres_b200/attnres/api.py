"""``attnres(values, query, *, eps, scale)``: the one public function.

Signature, defaults, accepted containers and the exceptions raised for bad arguments are those
of the reference's entry point (src/attnres/api.py:30-62); the work is done by the sm_100a
library behind ``attnres_b200::read_packed_forward`` / ``read_sources_forward``.
"""
from __future__ import annotations

from typing import Sequence, Union

import torch

from . import _sources

Values = Union[torch.Tensor, Sequence[torch.Tensor]]


def attnres(values: Values, query: torch.Tensor, *, eps: float = _sources.DEFAULT_EPS,
            scale: float = 1.0) -> torch.Tensor:
    """Softmax-over-sources read of ``values`` with the static ``query``.

    ``values``: one packed tensor ``[S, ..., D]``, or a list / tuple of ``S`` tensors
    ``[..., D]`` (any strides; nothing is stacked or copied unless a source's leading axes cannot
    be walked with one stride).  ``query``: ``[R]``, ``1 <= R <= D``.  The key of source ``s`` at
    a position is the RMS-normalised tail ``v_s[..., D-R:]`` (``eps`` inside the square root);
    its logit is ``scale`` times the key's dot product with ``query``; the result is the
    softmax-weighted sum of the full-width sources, one softmax per position.  ``R == D`` is the
    standard form, ``R < D`` the sliced low-rank one.

    Storage is BF16 on a CUDA device, arithmetic FP32; the result is BF16 ``[..., D]`` and
    carries first-order gradients to every source and to ``query``.
    """
    if torch.is_tensor(values):
        _sources.check_packed(values, query, eps, scale)
        from . import _ops  # deferred: loading the CUDA library is not needed to reject a call
        return _ops.packed_read(values, query, eps, scale)
    listed = _sources.check_sources(values, query, eps, scale)
    if listed[0].device.type != "cuda":
        raise RuntimeError("attnres requires CUDA tensors")
    from . import _ops
    return _ops.sources_read(listed, query, eps, scale)


__all__ = ["attnres"]
