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

from . import _ops
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


def _group_name(group) -> str:
    """Name of the process group for the functional all-reduce ("" = no collective)."""
    if not (dist.is_available() and dist.is_initialized()):
        return ""
    group = dist.group.WORLD if group is None else group
    return group.group_name if dist.get_world_size(group) > 1 else ""


def _sum_over_group(grad_fp32: torch.Tensor, group_name: str) -> torch.Tensor:
    """FP32 sum over the group (a traceable functional collective), rounded to BF16 once."""
    if group_name:
        import torch.distributed._functional_collectives as funcol
        grad_fp32 = funcol.all_reduce(grad_fp32, "sum", group_name)
    return grad_fp32.to(torch.bfloat16)


# Two torch.library operators (packed and list form): the forward is the local read; autograd
# runs the local backward with an FP32 query gradient and then the all-reduce.  They are
# opaque custom ops with fake kernels, like the plain read, so a sharded read traces under
# torch.compile(fullgraph=True).

@_ops._custom_op("attnres_b200::sharded_packed_forward", mutates_args=(), device_types="cuda")
def sharded_packed_forward(values: torch.Tensor, query: torch.Tensor, eps: float, scale: float,
                           group_name: str
                           ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    _ops._require_cuda_bf16((values,), query)
    kept, ptrs, row_strides, feat_strides = _ops._packed_table(values)
    return _ops._run_forward(kept, ptrs, row_strides, feat_strides, values.shape[1:], query, eps,
                             scale)


@sharded_packed_forward.register_fake
def _(values, query, eps, scale, group_name):
    rows = _ops._rows(values.shape[1:])
    keep = _ops._save_residual(values.shape[0], values.shape[-1], query.numel())
    return (values.new_empty(values.shape[1:]),
            values.new_empty((values.shape[0], rows), dtype=torch.float32),
            values.new_empty((2, rows), dtype=torch.float32),
            values.new_empty(values.shape[1:] if keep else (0,), dtype=torch.int16))


def _sharded_packed_setup(ctx, inputs, output) -> None:
    values, query, eps, scale, group_name = inputs
    out, logits, stats, residual = output
    ctx.mark_non_differentiable(logits, stats, residual)
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(values, query, logits, stats, out if residual.numel() else residual,
                          residual)
    ctx.eps, ctx.scale, ctx.group_name = eps, scale, group_name


def _sharded_packed_backward(ctx, grad_output, *_unused):
    if grad_output is None:
        return None, None, None, None, None
    values, query, logits, stats, out, residual = ctx.saved_tensors
    grad_values, grad_query = _ops.read_packed_backward(
        values, query, grad_output, logits, stats, out, residual, float(ctx.eps),
        float(ctx.scale), True, True, True)
    return grad_values, _sum_over_group(grad_query, ctx.group_name), None, None, None


torch.library.register_autograd(sharded_packed_forward, _sharded_packed_backward,
                                setup_context=_sharded_packed_setup)


@_ops._custom_op("attnres_b200::sharded_sources_forward", mutates_args=(), device_types="cuda",
                 **_ops._LIST_OP_KWARGS)
def sharded_sources_forward(sources: list[torch.Tensor], query: torch.Tensor, eps: float,
                            scale: float, group_name: str
                            ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    _ops._require_cuda_bf16(sources, query)
    kept, ptrs, row_strides, feat_strides = _ops._source_table(sources)
    return _ops._run_forward(kept, ptrs, row_strides, feat_strides, sources[0].shape, query, eps,
                             scale)


@sharded_sources_forward.register_fake
def _(sources, query, eps, scale, group_name):
    first = sources[0]
    rows = _ops._rows(first.shape)
    keep = _ops._save_residual(len(sources), first.shape[-1], query.numel())
    return (first.new_empty(first.shape),
            first.new_empty((len(sources), rows), dtype=torch.float32),
            first.new_empty((2, rows), dtype=torch.float32),
            first.new_empty(first.shape if keep else (0,), dtype=torch.int16))


def _sharded_sources_setup(ctx, inputs, output) -> None:
    sources, query, eps, scale, group_name = inputs
    out, logits, stats, residual = output
    ctx.mark_non_differentiable(logits, stats, residual)
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(*sources, query, logits, stats, out if residual.numel() else residual,
                          residual)
    ctx.count = len(sources)
    ctx.eps, ctx.scale, ctx.group_name = eps, scale, group_name


def _sharded_sources_backward(ctx, grad_output, *_unused):
    count = ctx.count
    if grad_output is None:
        return [None] * count, None, None, None, None
    saved = ctx.saved_tensors
    gradients = _ops.read_sources_backward(list(saved[:count]), saved[count], grad_output,
                                           saved[count + 1], saved[count + 2], saved[count + 3],
                                           saved[count + 4], float(ctx.eps), float(ctx.scale), True)
    return (gradients[:count], _sum_over_group(gradients[count], ctx.group_name), None, None, None)


torch.library.register_autograd(sharded_sources_forward, _sharded_sources_backward,
                                setup_context=_sharded_sources_setup)


def sharded_attnres(values, query: torch.Tensor, *, eps: float = DEFAULT_EPS, scale: float = 1.0,
                    group=None) -> torch.Tensor:
    """``attnres`` on this rank's rows; the query gradient is summed over ``group``.

    ``values`` holds only the rows this rank owns (see ``shard_rows``); ``query`` is
    replicated.  Every rank of the group must call this the same number of times, since
    the backward pass runs a collective.
    """
    name = _group_name(group)
    if isinstance(values, torch.Tensor):
        check_packed(values, query, eps, scale)
        if not values.is_cuda:
            raise RuntimeError("attnres requires CUDA tensors")
        return sharded_packed_forward(values, query, float(eps), float(scale), name)[0]
    sources = check_sources(values, query, eps, scale)
    if not sources[0].is_cuda:
        raise RuntimeError("attnres requires CUDA tensors")
    return sharded_sources_forward(list(sources), query, float(eps), float(scale), name)[0]


__all__ = ["all_reduce_query_grad", "shard_rows", "sharded_attnres"]
