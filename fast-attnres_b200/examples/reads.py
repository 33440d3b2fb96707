"""The AttnRes read in its four everyday forms: full-rank and sliced low-rank queries, packed and
list inputs, forward and backward.  Needs a CUDA device.

    python fast-attnres_b200/examples/reads.py

(The scenarios of the reference's examples standard_attnres.py, lr_attnres.py, packed_and_list.py
and backward.py, written for this package.)
"""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402

from attnres import LearnedQuery, attnres  # noqa: E402


def run(device: str = "cuda") -> dict:
    torch.manual_seed(1)
    sources, batch, tokens, width = 5, 2, 48, 256
    values = torch.randn(sources, batch, tokens, width, device=device, dtype=torch.bfloat16,
                         requires_grad=True)

    # full rank: the whole row is the key
    query = LearnedQuery(width).to(device)
    full = attnres(values, query())

    # sliced low rank: the last R coordinates are the key, the usual scale is 1/sqrt(R)
    rank = width // 4
    low = LearnedQuery(rank).to(device)
    sliced = attnres(values, low(), scale=rank ** -0.5)

    # an ordered list of separately allocated sources: no packing copy is made
    as_list = attnres([values[s] for s in range(sources)], query())
    assert torch.equal(as_list, full)

    # backward: BF16 gradients for the values, a gradient for the learned query
    upstream = torch.randn_like(full)
    grad_values, grad_query = torch.autograd.grad(full, (values, query.query), upstream)
    assert grad_values.shape == values.shape and grad_query.shape == (width,)
    return {"full": tuple(full.shape), "sliced": tuple(sliced.shape),
            "grad_values": str(grad_values.dtype), "grad_query": str(grad_query.dtype)}


if __name__ == "__main__":
    print(run())
