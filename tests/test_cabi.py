"""The C-ABI library: it loads, exports what the header declares, and rejects
bad arguments on the host (no kernel is launched by any test in this file)."""
import ctypes
import re
from pathlib import Path

import pytest

from attnres import _native

ROOT = Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "attnres_b200.h").read_text()


def _declared():
    names = set(re.findall(r"\b(attnres_b200_\w+)\s*\(", HEADER))
    assert names, "no declarations found in the header"
    return sorted(names)


def test_library_exports_every_declared_symbol():
    library = ctypes.CDLL(str(_native.LIBRARY_PATH))
    for name in _declared():
        assert hasattr(library, name), f"{name} is declared in the header but not exported"


def test_binding_covers_every_declared_symbol():
    assert sorted(_native.SIGNATURES) == _declared()


def test_abi_version_matches_header():
    version = int(re.search(r"#define ATTNRES_B200_ABI_VERSION (\d+)", HEADER).group(1))
    assert _native.load().attnres_b200_abi_version() == version == _native.ABI_VERSION


def test_status_strings():
    codes = {name: int(value) for name, value in
             re.findall(r"#define (ATTNRES_B200_(?:OK|ERR_\w+)) (\d+)", HEADER)}
    assert codes["ATTNRES_B200_OK"] == 0 and len(set(codes.values())) == len(codes)
    texts = {_native.status_text(code) for code in codes.values()}
    assert len(texts) == len(codes) and "unknown status" not in texts
    assert _native.status_text(999) == "unknown status"


def _forward_status(S=2, N=4, D=16, R=8, eps=2**-23, scale=1.0, src=0x1000, query=0x2000,
                    out=0x3000, logits=0x4000, stats=0x5000, flags=0):
    lib = _native.load()
    ptrs = _native.pointer_array([src] * max(S, 1))
    strides = _native.int64_array([D] * max(S, 1))
    ones = _native.int64_array([1] * max(S, 1))
    return lib.attnres_b200_forward(ptrs, strides, ones, S, N, D, R, query, 1, eps, scale,
                                    out, D, None, logits, stats, flags, None)


@pytest.mark.parametrize("kwargs,code", [
    (dict(S=0), 2), (dict(S=130), 2), (dict(D=0), 3), (dict(D=8193), 3),
    (dict(R=0), 4), (dict(R=17), 4), (dict(N=0), 5),
    (dict(eps=0.0), 6), (dict(eps=float("nan")), 6), (dict(scale=float("inf")), 6),
    (dict(query=None), 1), (dict(out=None), 1), (dict(logits=None), 1), (dict(stats=None), 1),
    (dict(src=None), 1), (dict(src=0x1001), 7), (dict(out=0x3001), 7), (dict(flags=64), 10),
])
def test_forward_argument_errors_are_found_before_any_launch(kwargs, code):
    assert _forward_status(**kwargs) == code


def test_backward_argument_errors_are_found_before_any_launch():
    lib = _native.load()
    S, N, D, R = 2, 4, 16, 8
    ptrs = _native.pointer_array([0x1000] * S)
    strides = _native.int64_array([D] * S)
    ones = _native.int64_array([1] * S)

    def call(S=S, go=0x6000, dsrc=ptrs, dstr=strides, partials=0x7000, rows=4, dq=0x8000,
             dq32=None, eps=2**-23):
        return lib.attnres_b200_backward(ptrs, strides, ones, S, N, D, R, 0x2000, 1, eps, 1.0,
                                         go, D, 1, 0x4000, 0x5000, None, None, dsrc, dstr, partials, rows,
                                         dq, dq32, 0, None)

    assert call(S=0) == 2
    assert call(eps=-1.0) == 6
    assert call(go=None) == 1
    assert call(dsrc=None, dstr=None, dq=None) == 11      # nothing to compute
    assert call(dstr=None) == 1
    assert call(partials=None) == 1
    assert call(dq=0x8001) == 7


def test_static_scratch_backward_checks_arguments_like_the_workspace_backward():
    """Same codes in the same order, found before the size limit or the device is looked at."""
    lib = _native.load()
    S, N, D, R = 2, 4, 16, 8
    ptrs = _native.pointer_array([0x1000] * S)
    strides = _native.int64_array([D] * S)
    ones = _native.int64_array([1] * S)

    def call(S=S, go=0x6000, dsrc=ptrs, dstr=strides, dq=0x8000, eps=2**-23, flags=0, R=R):
        return lib.attnres_b200_backward_static_scratch(
            ptrs, strides, ones, S, N, D, R, 0x2000, 1, eps, 1.0, go, D, 1, 0x4000, 0x5000,
            None, None, dsrc, dstr, dq, None, flags, None)

    assert call(S=0) == 2
    assert call(R=17) == 4
    assert call(eps=-1.0) == 6
    assert call(flags=64) == 10
    assert call(go=None) == 1
    assert call(dsrc=None, dstr=None, dq=None) == 11
    assert call(dstr=None) == 1
    assert call(dq=0x8001) == 7


def test_selftest_entry_point_checks_its_arguments():
    lib = _native.load()
    assert lib.attnres_b200_selftest_wait_limit(None, 1000000, None) == 1
    assert lib.attnres_b200_selftest_wait_limit(0x1008, 1000000, None) == 7
    assert lib.attnres_b200_selftest_wait_limit(0x1000, 10, None) == 6
    assert lib.attnres_b200_selftest_wait_limit(0x1000, 10**12, None) == 6


def test_output_residual_policy_is_a_pure_host_decision():
    # lists of up to four sources never want it; a position that fills an SM's shared
    # memory does, and so do full-width rows of 2048 and more with a full-rank query from five
    # sources up; at 1024 features the middle source counts stay with the staged kernel
    assert not _native.wants_output_residual(2, 1024, 1024)
    assert not _native.wants_output_residual(4, 4096, 4096)
    assert not _native.wants_output_residual(25, 1024, 1024)
    assert not _native.wants_output_residual(17, 1024, 1024)
    assert _native.wants_output_residual(5, 1024, 1024)
    assert not _native.wants_output_residual(5, 512, 512)
    assert _native.wants_output_residual(25, 2048, 2048)
    assert _native.wants_output_residual(9, 1024, 1024)
    assert _native.wants_output_residual(33, 1024, 1024)
    assert not _native.wants_output_residual(7, 4096, 1024)
    assert not _native.wants_output_residual(16, 4096, 1024)
    assert _native.wants_output_residual(25, 4096, 4096)
    assert _native.wants_output_residual(33, 2048, 512)
    assert _native.wants_output_residual(9, 2048, 2048)
    assert _native.wants_output_residual(49, 1024, 1024)
    assert _native.wants_output_residual(49, 2048, 2048)
    assert _native.wants_output_residual(49, 4096, 4096)
    assert _native.wants_output_residual(129, 8192, 8192)
    assert not _native.wants_output_residual(49, 3000, 127)     # not the aligned fast class
    assert not _native.wants_output_residual(0, 1024, 1024)


def test_workspace_rows_validates_shape():
    lib = _native.load()
    assert lib.attnres_b200_dq_workspace_rows(0, 2, 16, 8, 0) == -5
    assert lib.attnres_b200_dq_workspace_rows(4, 2, 16, 17, 0) == -4


def test_kernel_family_selection_is_a_pure_host_decision():
    from attnres import _native
    assert _native.kernel_family(9, 2048, 2048, True, False) == "tma"
    assert _native.kernel_family(9, 2048, 2048, True, True) == "tma"
    assert _native.kernel_family(16, 4096, 1024, True, True) == "tma"
    assert _native.kernel_family(9, 2048, 2048, False, True) == "generic"
    assert _native.kernel_family(9, 3000, 127, True, False) == "generic"
    assert _native.kernel_family(49, 4096, 4096, True, True) == "tma"       # a 2-CTA cluster shares the row
    # 2.1 MB per position: no staged kernel takes it, the one-pass kernel (whose forward saves
    # the output) does
    assert _native.kernel_family(129, 8192, 8192, True, True) == "tma"
    assert _native.wants_output_residual(129, 8192, 8192)
    assert _native.kernel_family(49, 4096, 4096, True, False) == "tma"
    assert _native.kernel_family(2, 1024, 1024, False, False) == "generic"
    assert _native.kernel_family(0, 1024, 1024, True, False) == "invalid"


def test_layer_norm_backward_entry_point_checks_its_arguments():
    lib = _native.load()

    def call(grad=0x1000, stride=16, out=0x2000, stats=0x3000, N=4, D=16, dx=0x4000,
             partials=0x5000, rows=4, both=0x6000):
        return lib.attnres_b200_layer_norm_backward(grad, stride, out, stats, None, N, D, dx,
                                                    partials, rows, both, None)

    assert call(D=0) == 3 and call(D=8200) == 3
    assert call(N=0) == 5
    assert call(grad=None) == 1 and call(both=None) == 1
    assert call(D=12) == 7            # rows of 12 features cannot be read 16 bytes at a time
    assert call(grad=0x1008) == 7 and call(stride=12) == 7
    assert lib.attnres_b200_layer_norm_workspace_rows(0, 16, 0) == -5
    assert lib.attnres_b200_layer_norm_workspace_rows(4, 0, 0) == -3
