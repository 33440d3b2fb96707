"""Position sharding of the AttnRes read across the GPUs of one node.

The softmax runs over the SOURCE axis independently at every position, so the
carried batch/token rows can be split across ranks with no communication in the
forward pass or in the value gradients.  The only exchange is the query
gradient: each rank reduces its rows to an FP32 ``[R]`` vector, the vectors are
summed with one all-reduce (NCCL over NVLink on GPUs, any backend in tests), and
the sum is rounded to BF16 once, so a G-rank result differs from the one-rank
result only by FP32 reassociation.  The reference has no distributed code; this
module is new.

When the query is a model parameter under data parallelism its gradient already
rides the framework's gradient all-reduce and plain ``attnres`` is enough; use
``sharded_attnres`` when one logical read is split across ranks.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ._sources import DEFAULT_EPS, check_packed, check_sources


def shard_rows(total_rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """Half-open row range ``[start, stop)`` owned by ``rank``: contiguous, ordered by
    rank, sizes differing by at most one (the first ``total_rows % world_size`` ranks
    take the extra row)."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank must satisfy 0 <= rank < world_size")
    if total_rows < 0:
        raise ValueError("total_rows must be non-negative")
    base, extra = divmod(total_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def all_reduce_query_grad(grad_fp32: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the per-rank FP32 query gradients in place and return the BF16 rounding."""
    if grad_fp32.dtype != torch.float32:
        raise TypeError("the cross-rank reduction runs on the FP32 query gradient")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(grad_fp32, op=dist.ReduceOp.SUM, group=group)
    return grad_fp32.to(torch.bfloat16)


class _ShardedRead(torch.autograd.Function):
    """Local forward; backward = local kernels with an FP32 query gradient, then all-reduce."""

    @staticmethod
    def forward(ctx, query, eps, scale, group, packed, *sources):
        from . import _ops
        if packed:
            kept, ptrs, rs, fs = _ops._packed_table(sources[0])
            shape = sources[0].shape[1:]
        else:
            kept, ptrs, rs, fs = _ops._source_table(sources)
            shape = sources[0].shape
        out, logits, stats, residual = _ops._run_forward(kept, ptrs, rs, fs, shape, query, eps,
                                                         scale)
        ctx.save_for_backward(query, logits, stats, out if residual.numel() else residual,
                              residual, *sources)
        ctx.eps, ctx.scale, ctx.group, ctx.packed = eps, scale, group, packed
        ctx.set_materialize_grads(False)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        from . import _ops
        count = len(ctx.saved_tensors) - 5
        if grad_output is None:
            return (None,) * (5 + count)
        query, logits, stats, out, residual, *sources = ctx.saved_tensors
        if ctx.packed:
            values = sources[0]
            kept, ptrs, rs, fs = _ops._packed_table(values)
            shape = values.shape[1:]
            grads = [torch.empty(tuple(values.shape), device=values.device, dtype=values.dtype)]
            step = grads[0].stride(0) * grads[0].element_size()
            grad_ptrs = [grads[0].data_ptr() + s * step for s in range(values.shape[0])]
        else:
            kept, ptrs, rs, fs = _ops._source_table(sources)
            shape = sources[0].shape
            grads = [torch.empty(tuple(shape), device=query.device, dtype=torch.bfloat16)
                     for _ in sources]
            grad_ptrs = [g.data_ptr() for g in grads]
        grad_query = _ops._run_backward(kept, ptrs, rs, fs, shape, query, grad_output, logits, stats,
                                        out, residual, ctx.eps, ctx.scale, grad_ptrs, True,
                                        query_grad_dtype=torch.float32)
        return (all_reduce_query_grad(grad_query, ctx.group), None, None, None, None, *grads)


def sharded_attnres(values, query: torch.Tensor, *, eps: float = DEFAULT_EPS, scale: float = 1.0,
                    group=None) -> torch.Tensor:
    """``attnres`` on this rank's rows; the query gradient is summed over ``group``.

    ``values`` holds only the rows this rank owns (see ``shard_rows``); ``query`` is
    replicated.  Every rank of the group must call this the same number of times, since
    the backward pass runs a collective.
    """
    if isinstance(values, torch.Tensor):
        check_packed(values, query, eps, scale)
        return _ShardedRead.apply(query, float(eps), float(scale), group, True, values)
    sources = check_sources(values, query, eps, scale)
    if not sources[0].is_cuda:
        raise RuntimeError("attnres requires CUDA tensors")
    return _ShardedRead.apply(query, float(eps), float(scale), group, False, *sources)


__all__ = ["all_reduce_query_grad", "shard_rows", "sharded_attnres"]
