"""AttnRes read whose backward ADDS the value gradients into caller-owned buffers.

In a network where every layer reads all earlier layer outputs (the Full schedule of the
reference's benchmark model, benchmarks/model.py:293-311), a source receives one gradient per
read that used it.  With the plain operator autograd materialises each per-read gradient and
then adds it to the running sum: three more passes over ``[N, D]`` per source and read (write
the gradient, read it back, read and write the sum).  A training loop that owns one running
gradient buffer per source can skip them: the kernels here read the buffer row, add this read's
gradient in FP32 and round to BF16 once (``dsrc[s] += dV_s``), so a read costs one read and one
write of the buffer instead of one write plus a separate accumulation pass.  The reference has
no such form; this module is new.

Usage::

    buffers = [torch.zeros_like(s) for s in sources]          # one per source, reused by every read
    out = attnres_accumulate(sources, query, buffers)         # forward: same result as attnres()
    out.backward(grad)                                        # buffers[s] += dV_s; query.grad as usual
    torch.autograd.backward(sources, grad_tensors=buffers)    # continue into the producers

The sources get NO gradient through autograd from this call (it is in the buffers).  The read
is a ``torch.library`` operator whose backward operator declares the buffers as mutated
arguments, so it runs eagerly, under CUDA graphs and under ``torch.compile``.
"""
from __future__ import annotations

import torch

from . import _native, _ops
from ._sources import DEFAULT_EPS, check_packed, check_sources


def _check_buffers(buffers, shapes, device) -> None:
    if len(buffers) != len(shapes):
        raise ValueError("one gradient buffer per source is required")
    for buffer, shape in zip(buffers, shapes):
        if not isinstance(buffer, torch.Tensor):
            raise TypeError("gradient buffers must be tensors")
        if buffer.dtype != torch.bfloat16:
            raise TypeError("gradient buffers must be BF16")
        if buffer.device != device:
            raise TypeError("gradient buffers must be on the sources' device")
        if tuple(buffer.shape) != tuple(shape):
            raise ValueError("a gradient buffer must have the shape of its source")
        if not buffer.is_contiguous():
            raise ValueError("gradient buffers must be contiguous")
        if buffer.requires_grad:
            raise ValueError("gradient buffers must not require grad")
    if not torch.compiler.is_compiling():   # addresses exist at run time only: the forward
        _check_no_overlap(buffers)           # operator repeats this check when it runs


def _check_no_overlap(buffers) -> None:
    """The kernels fetch a buffer row before they add to it: two sources whose buffers share
    any memory (the same tensor, or overlapping views of one storage) would lose an update."""
    spans = sorted((b.data_ptr(), b.data_ptr() + b.numel() * b.element_size()) for b in buffers)
    for (_, end), (start, _) in zip(spans, spans[1:]):
        if start < end:
            raise ValueError("every source needs its own gradient buffer (buffers overlap)")


# Two torch.library operators: the forward is the plain read (it always keeps the output and
# its residual: the accumulating backward of the fast layout class is the one-pass kernel);
# the backward operator declares the buffers as mutated arguments, so a read whose backward
# accumulates traces under torch.compile like any other in-place custom op.  The buffers ride
# along the forward operator only to reach its backward; the forward does not touch them.

@_ops._custom_op("attnres_b200::accumulate_sources_forward", mutates_args=(), device_types="cuda",
                 **_ops._LIST_OP_KWARGS)
def accumulate_sources_forward(sources: list[torch.Tensor], query: torch.Tensor,
                               buffers: list[torch.Tensor], eps: float, scale: float,
                               overwrite: bool
                               ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    _ops._require_cuda_bf16(sources, query)
    _check_no_overlap(buffers)
    kept, ptrs, rs, fs = _ops._source_table(sources)
    return _ops._run_forward(kept, ptrs, rs, fs, sources[0].shape, query, eps, scale,
                             keep_residual=True)


@accumulate_sources_forward.register_fake
def _(sources, query, buffers, eps, scale, overwrite):
    first = sources[0]
    rows = _ops._rows(first.shape)
    return (first.new_empty(first.shape),
            first.new_empty((len(sources), rows), dtype=torch.float32),
            first.new_empty((2, rows), dtype=torch.float32),
            first.new_empty(first.shape, dtype=torch.int16))


@_ops._custom_op("attnres_b200::accumulate_sources_backward", mutates_args=("buffers",),
                 device_types="cuda")
def accumulate_sources_backward(sources: list[torch.Tensor], query: torch.Tensor,
                                grad_output: torch.Tensor, logits: torch.Tensor,
                                stats: torch.Tensor, out: torch.Tensor, residual: torch.Tensor,
                                buffers: list[torch.Tensor], eps: float, scale: float,
                                overwrite: bool, need_query: bool) -> torch.Tensor:
    """buffers[s] += dV_s (or = dV_s with `overwrite`); returns the BF16 query gradient, or a
    0-element tensor when it is not needed."""
    _ops._require_cuda_bf16((*sources, grad_output, *buffers), query)
    kept, ptrs, rs, fs = _ops._source_table(sources)
    grad_query = _ops._run_backward(kept, ptrs, rs, fs, sources[0].shape, query, grad_output,
                                    logits, stats, out, residual, eps, scale,
                                    [b.data_ptr() for b in buffers], need_query,
                                    extra_flags=0 if overwrite else _native.FLAG_ACCUMULATE_DV)
    return grad_query if grad_query is not None else query.new_empty((0,))


@accumulate_sources_backward.register_fake
def _(sources, query, grad_output, logits, stats, out, residual, buffers, eps, scale, overwrite,
      need_query):
    return query.new_empty(query.shape if need_query else (0,))


def _accumulate_setup(ctx, inputs, output) -> None:
    sources, query, buffers, eps, scale, overwrite = inputs
    out, logits, stats, residual = output
    ctx.mark_non_differentiable(logits, stats, residual)
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(*sources, query, logits, stats, out, residual)
    # Not saved tensors: later reads' backwards update the buffers in place before this
    # read's backward runs, which autograd's version check would take for a bug.
    ctx.buffers = list(buffers)
    ctx.count = len(sources)
    ctx.eps, ctx.scale, ctx.overwrite = eps, scale, overwrite


def _accumulate_backward(ctx, grad_output, *_unused):
    count = ctx.count
    nothing = ([None] * count, None, [None] * count, None, None, None)
    if grad_output is None:
        return nothing
    saved = ctx.saved_tensors
    need_query = bool(ctx.needs_input_grad[1])
    grad_query = accumulate_sources_backward(
        list(saved[:count]), saved[count], grad_output, saved[count + 1], saved[count + 2],
        saved[count + 3], saved[count + 4], ctx.buffers, float(ctx.eps), float(ctx.scale),
        bool(ctx.overwrite), need_query)
    return ([None] * count, grad_query if need_query else None, [None] * count, None, None, None)


torch.library.register_autograd(accumulate_sources_forward, _accumulate_backward,
                                setup_context=_accumulate_setup)


def attnres_accumulate(values, query: torch.Tensor, grad_buffers, *, eps: float = DEFAULT_EPS,
                       scale: float = 1.0, overwrite: bool = False) -> torch.Tensor:
    """``attnres(values, query)`` whose backward adds dV into ``grad_buffers`` in place.

    ``overwrite=True`` makes the backward of THIS call store its gradients instead of adding
    them: for the read whose backward runs first in a step, so the buffers need no zeroing.

    ``values`` packed ``[S, ..., D]``: ``grad_buffers`` is one contiguous BF16 tensor of the
    same shape (read and updated through its S slices).  ``values`` a list/tuple of ``[..., D]``
    sources: ``grad_buffers`` is a list of contiguous BF16 tensors, one per source, each with
    its source's shape and its own memory.  The forward result and the query gradient are
    those of ``attnres``.
    """
    if isinstance(values, torch.Tensor):
        check_packed(values, query, eps, scale)
        if not values.is_cuda:
            raise RuntimeError("attnres requires CUDA tensors")
        if not isinstance(grad_buffers, torch.Tensor):
            raise TypeError("a packed call takes one packed gradient buffer")
        _check_buffers([grad_buffers], [values.shape], values.device)
        sources, buffers = list(values.unbind(0)), list(grad_buffers.unbind(0))
    else:
        sources = list(check_sources(values, query, eps, scale))
        if not sources[0].is_cuda:
            raise RuntimeError("attnres requires CUDA tensors")
        if not isinstance(grad_buffers, (list, tuple)):
            raise TypeError("a list call takes a list of gradient buffers")
        buffers = list(grad_buffers)
        _check_buffers(buffers, [s.shape for s in sources], sources[0].device)
    return accumulate_sources_forward(sources, query, buffers, float(eps), float(scale),
                                      bool(overwrite))[0]


__all__ = ["attnres_accumulate"]
