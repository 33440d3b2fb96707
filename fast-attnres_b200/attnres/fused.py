"""AttnRes read with the consumer's LayerNorm computed in the read's epilogue.

In the reference's model every read feeds a LayerNorm before the sublayer consumes it
(benchmarks/model.py:156, 170 of the reference); run separately, that LayerNorm reads the
``[N, D]`` result back from memory.  ``attnres_layer_norm`` returns the normalised row from the
same kernel that produced the read, while the row is still in registers.  The reference has no
such form; this module is new.

    normed = attnres_layer_norm(values, query, norm.weight, norm.bias, norm.eps)
    # == F.layer_norm(attnres(values, query).float(), (D,), weight, bias, eps) rounded to BF16

The normalisation is taken over the BF16-rounded read (what a separate LayerNorm would see) in
FP32.  It is a ``torch.library`` operator with a fake kernel and registered autograd, so it
traces under ``torch.compile(fullgraph=True)`` and captures into CUDA graphs; its backward is
two operators, the LayerNorm backward (from the saved read and the saved mean / rstd) and the
read's backward.
"""
from __future__ import annotations

import torch

from . import _native, _ops
from ._sources import DEFAULT_EPS, check_packed, check_sources


@_ops._custom_op("attnres_b200::read_sources_norm_forward", mutates_args=(), device_types="cuda",
                 **_ops._LIST_OP_KWARGS)
def read_sources_norm_forward(sources: list[torch.Tensor], query: torch.Tensor,
                              weight: torch.Tensor, bias: torch.Tensor, eps: float, scale: float,
                              norm_eps: float
                              ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                                         torch.Tensor, torch.Tensor]:
    """-> (normed, out, norm_stats [2,N], logits [S,N], stats [2,N], residual)."""
    _ops._require_cuda_bf16(sources, query)
    if weight.dtype != torch.float32 or bias.dtype != torch.float32:
        raise TypeError("LayerNorm weight and bias must be FP32")
    kept, ptrs, row_strides, feat_strides = _ops._source_table(sources)
    shape = sources[0].shape
    S, D, R, N = len(ptrs), int(shape[-1]), int(query.numel()), _ops._rows(shape)
    if weight.numel() != D or bias.numel() != D:
        raise ValueError("LayerNorm weight and bias must have the width of the sources")
    device = query.device
    weight, bias = weight.contiguous(), bias.contiguous()
    out = torch.empty(tuple(shape), device=device, dtype=torch.bfloat16)
    normed = torch.empty(tuple(shape), device=device, dtype=torch.bfloat16)
    norm_stats = torch.empty((2, N), device=device, dtype=torch.float32)
    logits = torch.empty((S, N), device=device, dtype=torch.float32)
    stats = torch.empty((2, N), device=device, dtype=torch.float32)
    keep = _ops._save_residual(S, D, R)
    residual = torch.empty(tuple(shape) if keep else (0,), device=device, dtype=torch.int16)
    with torch.cuda.device(device):
        _native.forward_layer_norm(
            ptrs, row_strides, feat_strides, S, N, D, R, query.data_ptr(), int(query.stride(0)),
            float(eps), float(scale), out.data_ptr(), D, logits.data_ptr(), stats.data_ptr(),
            weight.data_ptr(), bias.data_ptr(), float(norm_eps), normed.data_ptr(),
            norm_stats.data_ptr(), _ops._flags, _ops._stream(device),
            residual_ptr=residual.data_ptr() if keep else None)
    del kept
    return normed, out, norm_stats, logits, stats, residual


@read_sources_norm_forward.register_fake
def _(sources, query, weight, bias, eps, scale, norm_eps):
    first = sources[0]
    rows = _ops._rows(first.shape)
    keep = _ops._save_residual(len(sources), first.shape[-1], query.numel())
    return (first.new_empty(first.shape), first.new_empty(first.shape),
            first.new_empty((2, rows), dtype=torch.float32),
            first.new_empty((len(sources), rows), dtype=torch.float32),
            first.new_empty((2, rows), dtype=torch.float32),
            first.new_empty(first.shape if keep else (0,), dtype=torch.int16))


@_ops._custom_op("attnres_b200::layer_norm_backward", mutates_args=(), device_types="cuda")
def layer_norm_backward(grad_normed: torch.Tensor, out: torch.Tensor, norm_stats: torch.Tensor,
                        weight: torch.Tensor
                        ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward of the fused LayerNorm from what the forward saved: the BF16 read `out` and
    (mean, rstd) per row.  -> (gradient of `out` in BF16, weight gradient, bias gradient in
    FP32), computed by the library's LayerNorm-backward kernel (6 D bytes per row: the gradient
    and the read in, the input gradient out).  One opaque operator, so a compiled training
    step sees two operators per read in its backward: this one and the read's backward."""
    width = out.shape[-1]
    rows = norm_stats.shape[1]
    device = out.device
    grad_rows = grad_normed.reshape(rows, width)
    if grad_rows.stride(-1) != 1:
        grad_rows = grad_rows.contiguous()
    out_rows = out.reshape(rows, width).contiguous()
    through = torch.empty((rows, width), device=device, dtype=torch.bfloat16)
    both = torch.empty((2 * width,), device=device, dtype=torch.float32)
    with torch.cuda.device(device):
        partial_rows = _native.layer_norm_workspace_rows(rows, width, device.index)
        partials = torch.empty((partial_rows, 2 * width), device=device, dtype=torch.float32)
        status = _native.layer_norm_backward(
            grad_rows.data_ptr(), int(grad_rows.stride(0)), out_rows.data_ptr(),
            norm_stats.data_ptr(), weight.data_ptr(), rows, width, through.data_ptr(),
            partials.data_ptr(), partial_rows, both.data_ptr(), _ops._stream(device))
    if status == 0:
        return through.reshape(out.shape), both[:width].clone(), both[width:].clone()
    if status != _native.ERR_MISALIGNED:
        _native.check(status, "attnres_b200_layer_norm_backward")
    # A width or an alignment outside the kernel's: aten's LayerNorm backward on FP32 copies.
    mean = norm_stats[0].reshape(rows, 1)
    rstd = norm_stats[1].reshape(rows, 1)
    through, grad_weight, grad_bias = torch.ops.aten.native_layer_norm_backward(
        grad_normed.reshape(rows, width).float(), out.reshape(rows, width).float(), [width], mean,
        rstd, weight, weight, [True, True, True])   # the bias argument only lends its shape
    return through.to(torch.bfloat16).reshape(out.shape), grad_weight, grad_bias


@layer_norm_backward.register_fake
def _(grad_normed, out, norm_stats, weight):
    return (out.new_empty(out.shape), weight.new_empty(weight.shape),
            weight.new_empty(weight.shape))


def _setup(ctx, inputs, output) -> None:
    sources, query, weight, bias, eps, scale, norm_eps = inputs
    normed, out, norm_stats, logits, stats, residual = output
    ctx.mark_non_differentiable(norm_stats, logits, stats, residual)
    ctx.set_materialize_grads(False)
    # `out` is always kept: the LayerNorm backward needs it.
    ctx.save_for_backward(*sources, query, weight, norm_stats, logits, stats, out, residual)
    ctx.count = len(sources)
    ctx.eps, ctx.scale = eps, scale


def _backward(ctx, grad_normed, grad_out, *_unused):
    count = ctx.count
    nothing = ([None] * count, None, None, None, None, None, None)
    if grad_normed is None and grad_out is None:
        return nothing
    saved = ctx.saved_tensors
    sources, query, weight, norm_stats, logits, stats, out, residual = (
        list(saved[:count]), *saved[count:])
    grad_weight = grad_bias = None
    total = grad_out
    if grad_normed is not None:
        through, grad_weight, grad_bias = layer_norm_backward(grad_normed, out, norm_stats, weight)
        total = through if total is None else (total.float() + through.float()).to(torch.bfloat16)
    gradients = _ops.read_sources_backward(sources, query, total, logits, stats,
                                           out, residual, float(ctx.eps), float(ctx.scale), False)
    return gradients[:count], gradients[count], grad_weight, grad_bias, None, None, None


torch.library.register_autograd(read_sources_norm_forward, _backward, setup_context=_setup)


def attnres_layer_norm(values, query: torch.Tensor, weight: torch.Tensor | None = None,
                       bias: torch.Tensor | None = None, norm_eps: float = 1e-5, *,
                       eps: float = DEFAULT_EPS, scale: float = 1.0, return_read: bool = False):
    """``LayerNorm(attnres(values, query))`` over the last axis, from one kernel.

    ``values`` and ``query`` as for ``attnres`` (a packed ``[S, ..., D]`` tensor is read through
    its unbound sources).  ``weight`` / ``bias``: ``[D]`` tensors of any floating dtype (used in
    FP32), or None for ones / zeros.  Returns the normalised BF16 tensor, or
    ``(normed, read)`` with ``return_read=True``; both are differentiable.
    """
    if isinstance(values, torch.Tensor):
        check_packed(values, query, eps, scale)
        sources = list(values.unbind(0))
    else:
        sources = list(check_sources(values, query, eps, scale))
    if not sources[0].is_cuda:
        raise RuntimeError("attnres requires CUDA tensors")
    width = sources[0].shape[-1]
    device = sources[0].device
    weight = (torch.ones(width, device=device) if weight is None else weight).float()
    bias = (torch.zeros(width, device=device) if bias is None else bias).float()
    normed, out = read_sources_norm_forward(sources, query, weight, bias, float(eps), float(scale),
                                            float(norm_eps))[:2]
    return (normed, out) if return_read else normed


__all__ = ["attnres_layer_norm"]
