"""torch.library operators and autograd for the AttnRes read.

Two operator pairs in the ``attnres_b200::`` namespace (a different namespace
from the reference's ``attnres::`` so both can live in one process):

* ``read_packed_forward`` / ``read_packed_backward`` for a ``[S, ..., D]`` tensor
  (role of src/attnres/_kernels/fixed_tail.py:904-1088), and
* ``read_sources_forward`` / ``read_sources_backward`` for an ordered list of
  ``[..., D]`` tensors (role of src/attnres/_kernels/fixed_tail_sources.py:78-183).

Both are opaque custom ops with fake kernels and registered autograd, so they
trace under ``torch.compile(fullgraph=True)`` and capture into CUDA graphs: the
real implementations only read ``data_ptr()``/strides, allocate outputs with
``torch.empty`` and enqueue kernels on the current stream through the C ABI.
Sources are never stacked, concatenated or copied unless a source's leading
axes cannot be described by one row stride.
"""
from __future__ import annotations

import inspect
import math

import torch

from . import _native
from ._sources import _affine_row_stride, row_layout

_custom_op = torch.library.custom_op
_LIST_OP_KWARGS: dict = {}
if ("tags" in inspect.signature(_custom_op).parameters and hasattr(torch, "Tag")
        and hasattr(torch.Tag, "flexible_layout")):
    # Inductor may hand the list ops sources with other strides than eager did;
    # the implementations below honour whatever strides arrive.
    _LIST_OP_KWARGS = {"tags": (torch.Tag.flexible_layout,)}

# Test hook: OR-ed into the `flags` argument of every C-ABI call.
_flags = 0


def set_kernel_flags(flags: int) -> int:
    """Set the flag word passed to the library (0, FLAG_FORCE_GENERIC or FLAG_PREFER_STREAM);
    returns the old one."""
    global _flags
    previous, _flags = _flags, int(flags)
    return previous


def _save_residual(count: int, width: int, rank: int) -> bool:
    """Whether the forward also writes the 16-bit residual of its output.

    The library's one-pass backward for long source lists needs the forward's FP32 result
    (the BF16 output plus the 16 bits its rounding dropped, an int16 tensor of the output's
    shape); the decision depends on the shape only, so the fake kernels below make the same
    one.
    """
    return bool(_flags & _native.FLAG_PREFER_STREAM) or \
        _native.wants_output_residual(int(count), int(width), int(rank))


def _rows(shape) -> int:
    return int(math.prod(shape[:-1])) if len(shape) > 1 else 1


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda_bf16(tensors, query) -> None:
    if query.dtype != torch.bfloat16 or any(t.dtype != torch.bfloat16 for t in tensors):
        raise TypeError("attnres_b200 operators require BF16 storage")
    if not query.is_cuda or any(not t.is_cuda for t in tensors):
        raise RuntimeError("attnres_b200 operators require CUDA tensors")


def _require_saved_output(out, residual) -> None:
    """`out` is the forward's BF16 output when its int16 residual was written, else both are
    0-element stand-ins."""
    if residual.numel() and (out.dtype != torch.bfloat16 or residual.dtype != torch.int16
                             or out.shape != residual.shape):
        raise TypeError("the saved output must be BF16 with an int16 residual of the same shape")


def _source_table(sources):
    """(kept tensors, pointers, row strides, feature strides) for a source list."""
    kept, ptrs, row_strides, feat_strides = [], [], [], []
    for source in sources:
        tensor, row_stride, feat_stride = row_layout(source)
        kept.append(tensor)
        ptrs.append(tensor.data_ptr())
        row_strides.append(row_stride)
        feat_strides.append(feat_stride)
    return kept, ptrs, row_strides, feat_strides


def _packed_table(values):
    """Same for a packed [S, ..., D] tensor: one layout, S base addresses."""
    if _affine_row_stride(values[0]) is None:
        values = values.contiguous()
    _, row_stride, feat_stride = row_layout(values[0])
    count = values.shape[0]
    step = values.stride(0) * values.element_size()
    base = values.data_ptr()
    return values, [base + s * step for s in range(count)], [row_stride] * count, \
        [feat_stride] * count


def _run_forward(kept, ptrs, row_strides, feat_strides, shape, query, eps, scale,
                 keep_residual=None):
    S, D, R, N = len(ptrs), int(shape[-1]), int(query.numel()), _rows(shape)
    device = query.device
    out = torch.empty(tuple(shape), device=device, dtype=torch.bfloat16)
    logits = torch.empty((S, N), device=device, dtype=torch.float32)
    stats = torch.empty((2, N), device=device, dtype=torch.float32)
    # A 0-element residual means "not saved": the backward then takes the two-pass kernels.
    if keep_residual is None:
        keep_residual = _save_residual(S, D, R)
    residual = torch.empty(tuple(shape) if keep_residual else (0,), device=device,
                           dtype=torch.int16)
    with torch.cuda.device(device):
        _native.forward(ptrs, row_strides, feat_strides, S, N, D, R,
                        query.data_ptr(), int(query.stride(0)), float(eps), float(scale),
                        out.data_ptr(), D, logits.data_ptr(), stats.data_ptr(),
                        _flags, _stream(device),
                        residual_ptr=residual.data_ptr() if residual.numel() else None)
    del kept
    return out, logits, stats, residual


def _run_backward(kept, ptrs, row_strides, feat_strides, shape, query, grad_output, logits,
                  stats, out, residual, eps, scale, grad_ptrs, need_query,
                  query_grad_dtype=torch.bfloat16, extra_flags=0):
    S, D, R, N = len(ptrs), int(shape[-1]), int(query.numel()), _rows(shape)
    device = query.device
    upstream, go_row_stride, go_feat_stride = row_layout(grad_output.reshape(tuple(shape)))
    partials = grad_query = None
    partial_rows = 0
    saved = residual.numel() > 0 and out.is_contiguous() and residual.is_contiguous()
    with torch.cuda.device(device):
        if need_query:
            partial_rows = _native.dq_workspace_rows(N, S, D, R, device.index)
            partials = torch.empty((partial_rows, R), device=device, dtype=torch.float32)
            grad_query = torch.empty((R,), device=device, dtype=query_grad_dtype)
        as_f32 = query_grad_dtype == torch.float32
        _native.backward(
            ptrs, row_strides, feat_strides, S, N, D, R,
            query.data_ptr(), int(query.stride(0)), float(eps), float(scale),
            upstream.data_ptr(), go_row_stride, go_feat_stride,
            logits.data_ptr(), stats.data_ptr(),
            grad_ptrs, None if grad_ptrs is None else [D] * S,
            None if partials is None else partials.data_ptr(), partial_rows,
            grad_query.data_ptr() if need_query and not as_f32 else None,
            grad_query.data_ptr() if need_query and as_f32 else None,
            _flags | extra_flags, _stream(device),
            out_ptr=out.data_ptr() if saved else None,
            residual_ptr=residual.data_ptr() if saved else None)
    del kept, upstream
    return grad_query


# --------------------------------------------------------------------------- packed

@_custom_op("attnres_b200::read_packed_forward", mutates_args=(), device_types="cuda")
def read_packed_forward(values: torch.Tensor, query: torch.Tensor, eps: float, scale: float
                        ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    _require_cuda_bf16((values,), query)
    kept, ptrs, row_strides, feat_strides = _packed_table(values)
    return _run_forward(kept, ptrs, row_strides, feat_strides, values.shape[1:], query, eps, scale)


@read_packed_forward.register_fake
def _(values, query, eps, scale):
    rows = _rows(values.shape[1:])
    keep = _save_residual(values.shape[0], values.shape[-1], query.numel())
    return (values.new_empty(values.shape[1:]),
            values.new_empty((values.shape[0], rows), dtype=torch.float32),
            values.new_empty((2, rows), dtype=torch.float32),
            values.new_empty(values.shape[1:] if keep else (0,), dtype=torch.int16))


@_custom_op("attnres_b200::read_packed_backward", mutates_args=(), device_types="cuda")
def read_packed_backward(values: torch.Tensor, query: torch.Tensor, grad_output: torch.Tensor,
                         logits: torch.Tensor, stats: torch.Tensor, out: torch.Tensor,
                         residual: torch.Tensor, eps: float, scale: float,
                         need_values: bool, need_query: bool, query_grad_fp32: bool
                         ) -> tuple[torch.Tensor, torch.Tensor]:
    """`query_grad_fp32`: return the query gradient as the FP32 second-stage sum (for a caller
    that adds it across ranks before the one rounding to BF16)."""
    _require_cuda_bf16((values, grad_output), query)
    _require_saved_output(out, residual)
    kept, ptrs, row_strides, feat_strides = _packed_table(values)
    shape = values.shape[1:]
    count, rows, width = values.shape[0], _rows(shape), int(shape[-1])
    grad_values = grad_ptrs = None
    if need_values:
        grad_values = torch.empty(tuple(values.shape), device=values.device, dtype=values.dtype)
        step = rows * width * values.element_size()
        grad_ptrs = [grad_values.data_ptr() + s * step for s in range(count)]
    grad_query = _run_backward(kept, ptrs, row_strides, feat_strides, shape, query, grad_output,
                               logits, stats, out, residual, eps, scale, grad_ptrs, need_query,
                               query_grad_dtype=torch.float32 if query_grad_fp32 else torch.bfloat16)
    # Schema outputs are plain tensors: an unused gradient is a 0-element stand-in.
    if grad_values is None:
        grad_values = values.new_empty((0,))
    if grad_query is None:
        grad_query = query.new_empty((0,))
    return grad_values, grad_query


@read_packed_backward.register_fake
def _(values, query, grad_output, logits, stats, out, residual, eps, scale, need_values,
      need_query, query_grad_fp32):
    return (values.new_empty(values.shape if need_values else (0,)),
            query.new_empty(query.shape if need_query else (0,),
                            dtype=torch.float32 if query_grad_fp32 else query.dtype))


def _packed_setup(ctx, inputs, output) -> None:
    values, query, eps, scale = inputs
    out, logits, stats, residual = output
    ctx.mark_non_differentiable(logits, stats, residual)
    ctx.set_materialize_grads(False)
    # The output itself is kept only when its residual was written (0 elements otherwise).
    ctx.save_for_backward(values, query, logits, stats, out if residual.numel() else residual,
                          residual)
    ctx.eps, ctx.scale = eps, scale


def _packed_backward(ctx, grad_output, _grad_logits=None, _grad_stats=None, _grad_residual=None):
    if grad_output is None:
        return None, None, None, None
    values, query, logits, stats, out, residual = ctx.saved_tensors
    need_values, need_query = bool(ctx.needs_input_grad[0]), bool(ctx.needs_input_grad[1])
    if not (need_values or need_query):
        return None, None, None, None
    grad_values, grad_query = read_packed_backward(
        values, query, grad_output, logits, stats, out, residual, float(ctx.eps),
        float(ctx.scale), need_values, need_query, False)
    return (grad_values if need_values else None, grad_query if need_query else None, None, None)


torch.library.register_autograd(read_packed_forward, _packed_backward, setup_context=_packed_setup)


# --------------------------------------------------------------------------- source lists

@_custom_op("attnres_b200::read_sources_forward", mutates_args=(), device_types="cuda",
            **_LIST_OP_KWARGS)
def read_sources_forward(sources: list[torch.Tensor], query: torch.Tensor, eps: float, scale: float
                         ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    _require_cuda_bf16(sources, query)
    kept, ptrs, row_strides, feat_strides = _source_table(sources)
    return _run_forward(kept, ptrs, row_strides, feat_strides, sources[0].shape, query, eps, scale)


@read_sources_forward.register_fake
def _(sources, query, eps, scale):
    first = sources[0]
    rows = _rows(first.shape)
    keep = _save_residual(len(sources), first.shape[-1], query.numel())
    return (first.new_empty(first.shape),
            first.new_empty((len(sources), rows), dtype=torch.float32),
            first.new_empty((2, rows), dtype=torch.float32),
            first.new_empty(first.shape if keep else (0,), dtype=torch.int16))


@_custom_op("attnres_b200::read_sources_backward", mutates_args=(), device_types="cuda",
            **_LIST_OP_KWARGS)
def read_sources_backward(sources: list[torch.Tensor], query: torch.Tensor,
                          grad_output: torch.Tensor, logits: torch.Tensor, stats: torch.Tensor,
                          out: torch.Tensor, residual: torch.Tensor,
                          eps: float, scale: float, query_grad_fp32: bool) -> list[torch.Tensor]:
    """Returns the S value gradients followed by the query gradient (FP32 second-stage sum
    when `query_grad_fp32`, else BF16)."""
    _require_cuda_bf16((*sources, grad_output), query)
    _require_saved_output(out, residual)
    kept, ptrs, row_strides, feat_strides = _source_table(sources)
    shape = sources[0].shape
    grads = [torch.empty(tuple(shape), device=query.device, dtype=torch.bfloat16)
             for _ in sources]
    grad_query = _run_backward(kept, ptrs, row_strides, feat_strides, shape, query, grad_output,
                               logits, stats, out, residual, eps, scale,
                               [g.data_ptr() for g in grads], True,
                               query_grad_dtype=torch.float32 if query_grad_fp32 else torch.bfloat16)
    return [*grads, grad_query]


@read_sources_backward.register_fake
def _(sources, query, grad_output, logits, stats, out, residual, eps, scale, query_grad_fp32):
    return [source.new_empty(source.shape) for source in sources] + [
        query.new_empty(query.shape, dtype=torch.float32 if query_grad_fp32 else query.dtype)]


def _sources_setup(ctx, inputs, output) -> None:
    sources, query, eps, scale = inputs
    out, logits, stats, residual = output
    ctx.mark_non_differentiable(logits, stats, residual)
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(*sources, query, logits, stats, out if residual.numel() else residual,
                          residual)
    ctx.count = len(sources)
    ctx.eps, ctx.scale = eps, scale


def _sources_backward(ctx, grad_output, _grad_logits=None, _grad_stats=None, _grad_residual=None):
    if grad_output is None:
        return [None] * ctx.count, None, None, None
    saved = ctx.saved_tensors
    count = ctx.count
    gradients = read_sources_backward(list(saved[:count]), saved[count], grad_output,
                                      saved[count + 1], saved[count + 2], saved[count + 3],
                                      saved[count + 4], float(ctx.eps), float(ctx.scale), False)
    return gradients[:count], gradients[count], None, None


torch.library.register_autograd(read_sources_forward, _sources_backward,
                                setup_context=_sources_setup)


def packed_read(values: torch.Tensor, query: torch.Tensor, eps: float, scale: float):
    return read_packed_forward(values, query, float(eps), float(scale))[0]


def sources_read(sources, query: torch.Tensor, eps: float, scale: float):
    return read_sources_forward(list(sources), query, float(eps), float(scale))[0]
