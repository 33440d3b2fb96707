"""CPU oracle for the AttnRes read.  TEST INFRASTRUCTURE ONLY.

This module is the checker the parity tests, the smoke run and the benchmark's
CPU-baseline leg compare against.  Nothing in the shipped package imports it and
the CUDA path never falls back to it.

Two restatements of the reference's definition (validation/oracle.py:5-19):

* ``oracle``            -- PyTorch, FP32 arithmetic on BF16-rounded inputs, BF16
                           result; gradients come from autograd.  It performs the
                           same tensor operations in the same order as the
                           reference oracle, so on one machine the two agree bit
                           for bit (pinned by tests/golden/reference_oracle.npz,
                           which was generated from the reference itself).
* ``closed_form``       -- NumPy float64 forward and hand-derived backward (the
                           equations the reference kernels implement,
                           src/attnres/_kernels/fixed_tail.py:606-864), used to
                           cross-check autograd and the C port.

Parity status: pinned (golden vectors from the reference oracle plus the
reference's analytic known-answer cases, tests/test_routing_checks.py:10-47 and
tests/test_softmax_stats.py:6-15 of the reference).
"""
from __future__ import annotations

import numpy as np
import torch


def oracle(values, query, *, eps: float = 2**-23, scale: float = 1.0) -> torch.Tensor:
    """BF16 in, FP32 inside, BF16 out (validation/oracle.py:5-19).

    ``values`` is a packed ``[S, ..., D]`` tensor or a list/tuple of ``[..., D]``
    tensors; ``query`` is ``[R]``.  Ambient autocast is switched off so the
    arithmetic does not depend on the caller's context.
    """
    as_list = isinstance(values, (list, tuple))
    every = (*values, query) if as_list else (values, query)
    if any(t.dtype != torch.bfloat16 for t in every):
        raise TypeError("the oracle requires BF16 tensors")
    rank = query.numel()
    with torch.autocast(device_type=query.device.type, enabled=False):
        stacked = torch.stack(tuple(values)) if as_list else values
        wide = stacked.float()                                   # [S, ..., D]
        tail = stacked[..., -rank:].float()                      # [S, ..., R]
        inv_rms = torch.rsqrt(tail.square().mean(-1, keepdim=True) + eps)
        logits = (tail * inv_rms * query.float()).sum(-1) * scale  # [S, ...]
        weights = logits.softmax(0)
        return (weights.unsqueeze(-1) * wide).sum(0).to(torch.bfloat16)


def oracle_with_grads(values, query, upstream, *, eps: float = 2**-23, scale: float = 1.0):
    """(out, dV, dq) of ``oracle`` for a packed BF16 ``values`` and BF16 ``upstream``."""
    v = values.detach().clone().requires_grad_()
    q = query.detach().clone().requires_grad_()
    out = oracle(v, q, eps=eps, scale=scale)
    dv, dq = torch.autograd.grad(out, (v, q), upstream)
    return out.detach(), dv, dq


def closed_form(values: np.ndarray, query: np.ndarray, upstream: np.ndarray | None = None, *,
                eps: float = 2**-23, scale: float = 1.0, logits: np.ndarray | None = None):
    """Float64 forward (and backward when ``upstream`` is given) on ``[S, N, D]`` arrays.

    ``logits`` (``[S, N]``) replaces the computed logits z when given.  Where one FP32
    ulp of a logit is not small against 1 (|z| > 1e6), two correct FP32 evaluations of z
    give visibly different softmax weights; passing a kernel's own saved logits checks
    everything downstream of them exactly.

    Returns ``out`` or ``(out, dV, dq)``, all float64 and un-rounded:

        t = v[..., D-R:]; r = 1/sqrt(mean(t^2) + eps); k = t*r; z = scale * k.q
        p = softmax_s(z); out = sum_s p_s v_s
        dw_s = v_s . dO; delta = sum_s p_s dw_s; dz_s = p_s (dw_s - delta)
        dq   = sum_{n,s} scale dz_s k_s
        dV_s = p_s dO + [tail] r_s (scale dz_s q - k_s dz_s z_s / R)
    """
    v = np.asarray(values, dtype=np.float64)
    q = np.asarray(query, dtype=np.float64)
    rank = q.shape[0]
    tail = v[..., -rank:]
    r = 1.0 / np.sqrt((tail * tail).mean(-1) + eps)             # [S, N]
    k = tail * r[..., None]
    z = scale * (k * q).sum(-1) if logits is None else np.asarray(logits, dtype=np.float64)
    z_shift = z - z.max(0, keepdims=True)
    p = np.exp(z_shift)
    p /= p.sum(0, keepdims=True)
    out = (p[..., None] * v).sum(0)
    if upstream is None:
        return out
    g = np.asarray(upstream, dtype=np.float64)                  # [N, D]
    dw = (v * g[None]).sum(-1)                                  # [S, N]
    delta = (p * dw).sum(0, keepdims=True)
    dz = p * (dw - delta)
    dq = (scale * dz[..., None] * k).sum((0, 1))
    dv = p[..., None] * g[None]
    dv = dv.copy()
    dv[..., -rank:] += r[..., None] * (scale * dz[..., None] * q - k * (dz * z / rank)[..., None])
    return out, dv, dq


def closed_form_dquery(values: torch.Tensor, query: torch.Tensor, upstream: torch.Tensor, *,
                       eps: float = 2**-23, scale: float = 1.0, block_rows: int = 256
                       ) -> torch.Tensor:
    """Float64 query gradient of ``closed_form`` for ``[S, N, D]`` tensors on any device,
    accumulated over blocks of rows so that large shapes need little memory.  The yardstick
    for an FP32 query gradient: FP32 results differ from it by accumulated rounding only."""
    rank = query.numel()
    q = query.double()
    total = torch.zeros(rank, dtype=torch.float64, device=values.device)
    for first in range(0, values.shape[1], block_rows):
        v = values[:, first:first + block_rows].double()
        g = upstream[first:first + block_rows].double()
        tail = v[..., -rank:]
        r = torch.rsqrt(tail.square().mean(-1) + eps)            # [S, n]
        k = tail * r[..., None]
        z = scale * (k * q).sum(-1)
        p = torch.softmax(z, 0)
        dw = (v * g[None]).sum(-1)
        dz = p * (dw - (p * dw).sum(0, keepdim=True))
        total += scale * torch.einsum("sn,snr->r", dz, k)
    return total


def join_saved_output(out: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """The FP32 result the forward kernels computed, from the BF16 output and the 16-bit
    residual they save with it (held in an int16 tensor, read as unsigned):
    float_bits = ((bf16_bits(out) << 16) | residual) - 0x8000."""
    high = out.contiguous().view(torch.int16).to(torch.int32) << 16
    low = residual.to(torch.int32) & 0xFFFF
    return ((high | low) - 0x8000).view(torch.float32)


def bf16_bits(tensor: torch.Tensor) -> np.ndarray:
    """The raw 16-bit patterns of a BF16 tensor as a uint16 array."""
    return tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def from_bf16_bits(bits: np.ndarray) -> torch.Tensor:
    """Inverse of ``bf16_bits``."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


def error_metrics(actual: torch.Tensor, expected: torch.Tensor) -> dict:
    """``max_abs`` and ``relative_l2`` exactly as validation/comparison.py:9-12 defines them."""
    difference = (actual.detach().float() - expected.detach().float()).abs()
    norm = torch.linalg.vector_norm(expected.detach().float()).clamp_min(1e-20)
    return {"max_abs": float(difference.max()),
            "relative_l2": float(torch.linalg.vector_norm(difference) / norm)}
