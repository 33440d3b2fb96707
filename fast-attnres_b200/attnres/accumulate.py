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

The sources get NO gradient through autograd from this call (it is in the buffers).  Eager and
CUDA-graph use only: the buffers are side effects, which ``torch.compile`` does not trace.
"""
from __future__ import annotations

import torch

from . import _native
from ._sources import DEFAULT_EPS, check_packed, check_sources


def _check_buffers(buffers, shapes, device) -> None:
    if len(buffers) != len(shapes):
        raise ValueError("one gradient buffer per source is required")
    spans = []
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
        spans.append((buffer.data_ptr(), buffer.data_ptr() + buffer.numel() * buffer.element_size()))
    # The kernels fetch a buffer row before they add to it: two sources whose buffers share
    # any memory (the same tensor, or overlapping views of one storage) would lose an update.
    spans.sort()
    for (_, end), (start, _) in zip(spans, spans[1:]):
        if start < end:
            raise ValueError("every source needs its own gradient buffer (buffers overlap)")


class _AccumulatingRead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, eps, scale, packed, buffers, overwrite, *sources):
        from . import _ops
        if packed:
            kept, ptrs, rs, fs = _ops._packed_table(sources[0])
            shape = sources[0].shape[1:]
        else:
            kept, ptrs, rs, fs = _ops._source_table(sources)
            shape = sources[0].shape
        # The output is always kept with its residual: the accumulating backward of the fast
        # layout class is the one-pass kernel (other layouts use the generic kernel and ignore it).
        out, logits, stats, residual = _ops._run_forward(kept, ptrs, rs, fs, shape, query, eps,
                                                         scale, keep_residual=True)
        ctx.save_for_backward(query, logits, stats, out, residual, *sources)
        ctx.eps, ctx.scale, ctx.packed, ctx.buffers = eps, scale, packed, buffers
        ctx.overwrite = overwrite
        ctx.set_materialize_grads(False)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        from . import _ops
        count = len(ctx.saved_tensors) - 5
        nothing = (None,) * (6 + count)
        if grad_output is None:
            return nothing
        query, logits, stats, out, residual, *sources = ctx.saved_tensors
        if ctx.packed:
            values = sources[0]
            kept, ptrs, rs, fs = _ops._packed_table(values)
            shape = values.shape[1:]
            buffer = ctx.buffers[0]
            step = buffer.stride(0) * buffer.element_size()
            grad_ptrs = [buffer.data_ptr() + s * step for s in range(values.shape[0])]
        else:
            kept, ptrs, rs, fs = _ops._source_table(sources)
            shape = sources[0].shape
            grad_ptrs = [b.data_ptr() for b in ctx.buffers]
        grad_query = _ops._run_backward(kept, ptrs, rs, fs, shape, query, grad_output, logits, stats,
                                        out, residual, ctx.eps, ctx.scale, grad_ptrs,
                                        bool(ctx.needs_input_grad[0]),
                                        extra_flags=0 if ctx.overwrite else _native.FLAG_ACCUMULATE_DV)
        return (grad_query, *nothing[1:])


def attnres_accumulate(values, query: torch.Tensor, grad_buffers, *, eps: float = DEFAULT_EPS,
                       scale: float = 1.0, overwrite: bool = False) -> torch.Tensor:
    """``attnres(values, query)`` whose backward adds dV into ``grad_buffers`` in place.

    ``overwrite=True`` makes the backward of THIS call store its gradients instead of adding
    them: for the read whose backward runs first in a step, so the buffers need no zeroing.

    ``values`` packed ``[S, ..., D]``: ``grad_buffers`` is one contiguous BF16 tensor of the
    same shape.  ``values`` a list/tuple of ``[..., D]`` sources: ``grad_buffers`` is a list of
    contiguous BF16 tensors, one per source, each with its source's shape and its own memory.
    The forward result and the query gradient are those of ``attnres``.
    """
    if isinstance(values, torch.Tensor):
        check_packed(values, query, eps, scale)
        if not values.is_cuda:
            raise RuntimeError("attnres requires CUDA tensors")
        if not isinstance(grad_buffers, torch.Tensor):
            raise TypeError("a packed call takes one packed gradient buffer")
        _check_buffers([grad_buffers], [values.shape], values.device)
        return _AccumulatingRead.apply(query, float(eps), float(scale), True, [grad_buffers],
                                       bool(overwrite), values)
    sources = check_sources(values, query, eps, scale)
    if not sources[0].is_cuda:
        raise RuntimeError("attnres requires CUDA tensors")
    if not isinstance(grad_buffers, (list, tuple)):
        raise TypeError("a list call takes a list of gradient buffers")
    _check_buffers(list(grad_buffers), [s.shape for s in sources], sources[0].device)
    return _AccumulatingRead.apply(query, float(eps), float(scale), False, list(grad_buffers),
                                   bool(overwrite), *sources)


__all__ = ["attnres_accumulate"]
