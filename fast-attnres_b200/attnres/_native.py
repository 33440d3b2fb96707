"""ctypes binding of ``libattnres_b200.so`` (C ABI: include/attnres_b200.h).

There is no fallback: if the library is missing or the wrong version, every
call raises.  Build it with ``python fast-attnres_b200/build.py``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int32, c_int64, c_uint32, c_uint64, c_void_p
from pathlib import Path

ABI_VERSION = 3
FLAG_FORCE_GENERIC = 1
FLAG_PREFER_STREAM = 2
FLAG_ACCUMULATE_DV = 4
LIBRARY_PATH = Path(__file__).resolve().parent / "_lib" / "libattnres_b200.so"

_PTR_ARRAY = ctypes.POINTER(c_void_p)
_I64_ARRAY = ctypes.POINTER(c_int64)

# name -> (restype, argtypes); one entry per declaration in include/attnres_b200.h
SIGNATURES = {
    "attnres_b200_abi_version": (c_int32, []),
    "attnres_b200_status_string": (c_char_p, [c_int32]),
    "attnres_b200_kernel_family": (c_char_p, [c_int32, c_int32, c_int32, c_int32, c_int32]),
    "attnres_b200_dq_workspace_rows": (c_int32, [c_int64, c_int32, c_int32, c_int32, c_int32]),
    "attnres_b200_error_flag": (c_int32, [ctypes.POINTER(c_int32), c_int32]),
    "attnres_b200_selftest_wait_limit": (c_int32, [c_void_p, c_uint64, c_void_p]),
    "attnres_b200_forward": (c_int32, [
        _PTR_ARRAY, _I64_ARRAY, _I64_ARRAY,
        c_int32, c_int64, c_int32, c_int32,
        c_void_p, c_int64, c_float, c_float,
        c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
        c_uint32, c_void_p]),
    "attnres_b200_forward_layer_norm": (c_int32, [
        _PTR_ARRAY, _I64_ARRAY, _I64_ARRAY,
        c_int32, c_int64, c_int32, c_int32,
        c_void_p, c_int64, c_float, c_float,
        c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_float, c_void_p, c_void_p,
        c_uint32, c_void_p]),
    "attnres_b200_layer_norm_workspace_rows": (c_int32, [c_int64, c_int32, c_int32]),
    "attnres_b200_layer_norm_backward": (c_int32, [
        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int32,
        c_void_p, c_void_p, c_int32, c_void_p, c_void_p]),
    "attnres_b200_wants_output_residual": (c_int32, [c_int32, c_int32, c_int32]),
    "attnres_b200_backward_static_scratch": (c_int32, [
        _PTR_ARRAY, _I64_ARRAY, _I64_ARRAY,
        c_int32, c_int64, c_int32, c_int32,
        c_void_p, c_int64, c_float, c_float,
        c_void_p, c_int64, c_int64,
        c_void_p, c_void_p, c_void_p, c_void_p,
        _PTR_ARRAY, _I64_ARRAY,
        c_void_p, c_void_p,
        c_uint32, c_void_p]),
    "attnres_b200_backward": (c_int32, [
        _PTR_ARRAY, _I64_ARRAY, _I64_ARRAY,
        c_int32, c_int64, c_int32, c_int32,
        c_void_p, c_int64, c_float, c_float,
        c_void_p, c_int64, c_int64,
        c_void_p, c_void_p, c_void_p, c_void_p,
        _PTR_ARRAY, _I64_ARRAY,
        c_void_p, c_int32,
        c_void_p, c_void_p,
        c_uint32, c_void_p]),
}

_library = None


def load() -> ctypes.CDLL:
    """Load the shared library once and check its ABI version."""
    global _library
    if _library is not None:
        return _library
    if not LIBRARY_PATH.exists():
        raise RuntimeError(
            f"{LIBRARY_PATH} is missing: the sm_100a CUDA library has not been built "
            "(run `python fast-attnres_b200/build.py`); there is no fallback path")
    library = ctypes.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        function = getattr(library, name)
        function.restype = restype
        function.argtypes = argtypes
    found = library.attnres_b200_abi_version()
    if found != ABI_VERSION:
        raise RuntimeError(f"libattnres_b200.so has ABI {found}, binding expects {ABI_VERSION}")
    _library = library
    return library


def status_text(status: int) -> str:
    return load().attnres_b200_status_string(int(status)).decode()


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed: {status_text(status)} (status {status})")


def pointer_array(addresses) -> ctypes.Array:
    return (c_void_p * len(addresses))(*addresses)


def int64_array(values) -> ctypes.Array:
    return (c_int64 * len(values))(*values)


def forward(src_ptrs, row_strides, feat_strides, S, N, D, R, query_ptr, query_stride,
            eps, scale, out_ptr, out_row_stride, logits_ptr, stats_ptr, flags, stream,
            residual_ptr=None) -> None:
    status = load().attnres_b200_forward(
        pointer_array(src_ptrs), int64_array(row_strides), int64_array(feat_strides),
        S, N, D, R, query_ptr, query_stride, eps, scale,
        out_ptr, out_row_stride, residual_ptr, logits_ptr, stats_ptr, flags, stream)
    check(status, "attnres_b200_forward")


def forward_layer_norm(src_ptrs, row_strides, feat_strides, S, N, D, R, query_ptr, query_stride,
                       eps, scale, out_ptr, out_row_stride, logits_ptr, stats_ptr,
                       weight_ptr, bias_ptr, norm_eps, normed_ptr, norm_stats_ptr, flags, stream,
                       residual_ptr=None) -> None:
    status = load().attnres_b200_forward_layer_norm(
        pointer_array(src_ptrs), int64_array(row_strides), int64_array(feat_strides),
        S, N, D, R, query_ptr, query_stride, eps, scale,
        out_ptr, out_row_stride, residual_ptr, logits_ptr, stats_ptr,
        weight_ptr, bias_ptr, norm_eps, normed_ptr, norm_stats_ptr, flags, stream)
    check(status, "attnres_b200_forward_layer_norm")


ERR_MISALIGNED = 7


def layer_norm_workspace_rows(N, D, device_index) -> int:
    rows = load().attnres_b200_layer_norm_workspace_rows(N, D, device_index)
    if rows < 0:
        check(-rows, "attnres_b200_layer_norm_workspace_rows")
    return rows


def layer_norm_backward(grad_ptr, grad_row_stride, out_ptr, stats_ptr, weight_ptr, N, D,
                        grad_out_ptr, partials_ptr, partial_rows, grad_weight_bias_ptr,
                        stream) -> int:
    """Returns the status code (0 = enqueued; ERR_MISALIGNED = layout outside the kernel's)."""
    return load().attnres_b200_layer_norm_backward(
        grad_ptr, grad_row_stride, out_ptr, stats_ptr, weight_ptr, N, D, grad_out_ptr,
        partials_ptr, partial_rows, grad_weight_bias_ptr, stream)


def wants_output_residual(S, D, R) -> bool:
    """Whether the backward of this shape is faster with the forward's output and residual."""
    return bool(load().attnres_b200_wants_output_residual(S, D, R))


def dq_workspace_rows(N, S, D, R, device_index) -> int:
    rows = load().attnres_b200_dq_workspace_rows(N, S, D, R, device_index)
    if rows < 0:
        check(-rows, "attnres_b200_dq_workspace_rows")
    return rows


def backward(src_ptrs, row_strides, feat_strides, S, N, D, R, query_ptr, query_stride,
             eps, scale, go_ptr, go_row_stride, go_feat_stride, logits_ptr, stats_ptr,
             dsrc_ptrs, dsrc_row_strides, partials_ptr, partial_rows,
             dq_bf16_ptr, dq_f32_ptr, flags, stream, out_ptr=None, residual_ptr=None) -> None:
    status = load().attnres_b200_backward(
        pointer_array(src_ptrs), int64_array(row_strides), int64_array(feat_strides),
        S, N, D, R, query_ptr, query_stride, eps, scale,
        go_ptr, go_row_stride, go_feat_stride, logits_ptr, stats_ptr, out_ptr, residual_ptr,
        None if dsrc_ptrs is None else pointer_array(dsrc_ptrs),
        None if dsrc_row_strides is None else int64_array(dsrc_row_strides),
        partials_ptr, partial_rows, dq_bf16_ptr, dq_f32_ptr, flags, stream)
    check(status, "attnres_b200_backward")


STATIC_SCRATCH_FLOATS = 2424832
ERR_STATIC_SCRATCH = 12


def backward_static_scratch(src_ptrs, row_strides, feat_strides, S, N, D, R, query_ptr,
                            query_stride, eps, scale, go_ptr, go_row_stride, go_feat_stride,
                            logits_ptr, stats_ptr, dsrc_ptrs, dsrc_row_strides,
                            dq_bf16_ptr, dq_f32_ptr, flags, stream, out_ptr=None,
                            residual_ptr=None) -> int:
    """Backward for callers that cannot allocate the dquery workspace: the partial sums go
    to a fixed array inside the library.  Returns the status code (0 = enqueued) instead of
    raising, so a caller can fall back to ``backward`` on ERR_STATIC_SCRATCH.  The first
    call on a device must happen outside stream capture; concurrent calls race."""
    return load().attnres_b200_backward_static_scratch(
        pointer_array(src_ptrs), int64_array(row_strides), int64_array(feat_strides),
        S, N, D, R, query_ptr, query_stride, eps, scale,
        go_ptr, go_row_stride, go_feat_stride, logits_ptr, stats_ptr, out_ptr, residual_ptr,
        None if dsrc_ptrs is None else pointer_array(dsrc_ptrs),
        None if dsrc_row_strides is None else int64_array(dsrc_row_strides),
        dq_bf16_ptr, dq_f32_ptr, flags, stream)


def error_flag(clear: bool = False) -> int:
    """The sticky "a kernel gave up waiting" flag of the current device (synchronises)."""
    value = c_int32(0)
    check(load().attnres_b200_error_flag(ctypes.byref(value), int(clear)), "attnres_b200_error_flag")
    return int(value.value)


def selftest_wait_limit(scratch_ptr, limit_ns, stream) -> None:
    """Run the library's bounded-wait self-test: afterwards ``error_flag()`` reads 1."""
    check(load().attnres_b200_selftest_wait_limit(scratch_ptr, int(limit_ns), stream),
          "attnres_b200_selftest_wait_limit")


def kernel_family(S, D, R, aligned, backward_pass) -> str:
    return load().attnres_b200_kernel_family(S, D, R, int(aligned), int(backward_pass)).decode()
