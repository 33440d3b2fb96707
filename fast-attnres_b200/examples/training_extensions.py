"""The additions for training loops: the read with its consumer's LayerNorm fused into the
epilogue, and the read whose backward adds the value gradients into caller-owned buffers.
Needs a CUDA device.

    python fast-attnres_b200/examples/training_extensions.py
"""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

from attnres import attnres  # noqa: E402
from attnres.accumulate import attnres_accumulate  # noqa: E402
from attnres.fused import attnres_layer_norm  # noqa: E402


def run(device: str = "cuda") -> dict:
    torch.manual_seed(3)
    count, rows, width = 7, 128, 1024
    sources = [torch.randn(rows, width, device=device, dtype=torch.bfloat16) for _ in range(count)]
    query = (torch.randn(width, device=device, dtype=torch.bfloat16) * 0.1).requires_grad_()
    norm = torch.nn.LayerNorm(width).to(device)

    # LayerNorm(attnres(...)) from one kernel
    fused = attnres_layer_norm(sources, query, norm.weight, norm.bias, norm.eps)
    separate = F.layer_norm(attnres(sources, query).float(), (width,), norm.weight, norm.bias, norm.eps)
    torch.testing.assert_close(fused.float(), separate, rtol=2**-7, atol=2**-7)

    # two reads of the same sources: each backward ADDS its value gradients into the buffers,
    # so autograd never materialises or sums per-read gradients
    buffers = [torch.zeros_like(s) for s in sources]
    upstream = torch.randn(rows, width, device=device, dtype=torch.bfloat16)
    attnres_accumulate(sources, query, buffers, overwrite=True).backward(upstream)
    attnres_accumulate(sources, query, buffers).backward(upstream)
    leaves = [s.clone().requires_grad_() for s in sources]
    (attnres(leaves, query.detach()) * 2.0).backward(upstream)
    torch.testing.assert_close(buffers[0].float(), leaves[0].grad.float(), rtol=0.05, atol=0.05)
    return {"fused": tuple(fused.shape), "buffers": len(buffers)}


if __name__ == "__main__":
    print(run())
