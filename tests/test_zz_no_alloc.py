"""The backward entry point that needs no caller workspace (collected last on purpose).

`attnres_b200_backward_static_scratch` serves hosts that may not allocate device memory
when they call the operator (an arena-owning runtime, a plugin inside a captured region):
its dquery partial sums go to a fixed array inside the library.  The checks: through the
C ABI it gives the same gradients as `attnres_b200_backward` on two calls in a row that
share the array, and it refuses shapes beyond the array with a clear status.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _case(s, n, d, r, seed):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    values = torch.randn(s, n, d, device="cuda", dtype=BF16, generator=generator)
    query = (torch.randn(r, device="cuda", generator=generator) * 0.25).to(BF16)
    upstream = torch.randn(n, d, device="cuda", dtype=BF16, generator=generator)
    return values, query, upstream


def _both_backwards(values, query, upstream, flags):
    from attnres import _native
    s, n, d = values.shape
    r = query.numel()
    out = torch.empty(n, d, device="cuda", dtype=BF16)
    logits = torch.empty(s, n, device="cuda", dtype=torch.float32)
    stats = torch.empty(2, n, device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    step = n * d * 2
    src = [values.data_ptr() + i * step for i in range(s)]
    table = (src, [d] * s, [1] * s, s, n, d, r, query.data_ptr(), 1, 2**-23, 0.5)
    # With the one-pass kernel asked for, the forward also saves its output's residual and
    # both backwards are handed the pair.
    one_pass = bool(flags & _native.FLAG_PREFER_STREAM)
    residual = torch.empty(n, d, device="cuda", dtype=torch.int16) if one_pass else None
    saved = dict(out_ptr=out.data_ptr(), residual_ptr=residual.data_ptr()) if one_pass else {}
    _native.forward(*table, out.data_ptr(), d, logits.data_ptr(), stats.data_ptr(), flags, stream,
                    residual_ptr=saved.get("residual_ptr"))

    def outputs():
        grads = torch.full((s, n, d), float("nan"), device="cuda", dtype=BF16)
        return (grads, torch.full((r,), float("nan"), device="cuda", dtype=BF16),
                torch.full((r,), float("nan"), device="cuda", dtype=torch.float32),
                [grads.data_ptr() + i * step for i in range(s)])

    rows = _native.dq_workspace_rows(n, s, d, r, 0)
    workspace = torch.empty(rows, r, device="cuda", dtype=torch.float32)
    want_dv, want_dq, want_dq32, ptrs = outputs()
    _native.backward(*table, upstream.data_ptr(), d, 1, logits.data_ptr(), stats.data_ptr(),
                     ptrs, [d] * s, workspace.data_ptr(), rows, want_dq.data_ptr(),
                     want_dq32.data_ptr(), flags, stream, **saved)
    got_dv, got_dq, got_dq32, ptrs = outputs()
    status = _native.backward_static_scratch(
        *table, upstream.data_ptr(), d, 1, logits.data_ptr(), stats.data_ptr(), ptrs, [d] * s,
        got_dq.data_ptr(), got_dq32.data_ptr(), flags, stream, **saved)
    assert status == 0, _native.status_text(status)
    torch.cuda.synchronize()
    return (want_dv, want_dq, want_dq32), (got_dv, got_dq, got_dq32)


@pytest.mark.parametrize("flags", [0, 1, 2], ids=["auto", "generic", "one-pass"])
def test_static_scratch_backward_matches_workspace_backward_twice_in_a_row(flags):
    # Two different problems back to back: the second call finds the first one's partial
    # sums in the shared array and must not be affected by them.
    for shape, seed in (((5, 777, 1024, 1024), 1), ((3, 2050, 512, 128), 2),
                        ((5, 777, 1024, 1024), 3)):
        values, query, upstream = _case(*shape, seed)
        want, got = _both_backwards(values, query, upstream, flags)
        for expected, actual in zip(want, got):
            assert torch.isfinite(actual.float()).all()
            # the tolerance of the parity tests ...
            torch.testing.assert_close(actual, expected, rtol=0.05, atol=0.05)
            # ... and, since both entry points run the same kernels over the same number
            # of partial rows, the same bits
            assert torch.equal(actual, expected)


def test_static_scratch_refuses_shapes_beyond_the_array_without_launching():
    from attnres import _native
    s, n, d, r = 1, 2048, 4096, 4096
    rows = _native.dq_workspace_rows(n, s, d, r, 0)
    assert rows * r > _native.STATIC_SCRATCH_FLOATS
    values, query, upstream = _case(s, n, d, r, 4)
    grads = torch.full((s, n, d), 3.0, device="cuda", dtype=BF16)
    dq = torch.full((r,), 3.0, device="cuda", dtype=BF16)
    logits = torch.zeros(s, n, device="cuda", dtype=torch.float32)
    stats = torch.ones(2, n, device="cuda", dtype=torch.float32)
    status = _native.backward_static_scratch(
        [values.data_ptr()], [d], [1], s, n, d, r, query.data_ptr(), 1, 2**-23, 1.0,
        upstream.data_ptr(), d, 1, logits.data_ptr(), stats.data_ptr(), [grads.data_ptr()], [d],
        dq.data_ptr(), None, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status == _native.ERR_STATIC_SCRATCH
    assert "scratch" in _native.status_text(status)
    assert bool((grads == 3.0).all()) and bool((dq == 3.0).all()), "a refused call wrote output"


def test_static_scratch_backward_without_query_gradient_needs_no_scratch():
    """Value gradients only: the call uses no scratch, so a shape whose query-gradient partials
    would not fit the array is served all the same."""
    from attnres import _native
    s, n, d, r = 2, 1500, 4096, 4096
    assert _native.dq_workspace_rows(n, s, d, r, 0) * r > _native.STATIC_SCRATCH_FLOATS
    values, query, upstream = _case(s, n, d, r, 5)
    out = torch.empty(n, d, device="cuda", dtype=BF16)
    logits = torch.empty(s, n, device="cuda", dtype=torch.float32)
    stats = torch.empty(2, n, device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    step = n * d * 2
    src = [values.data_ptr() + i * step for i in range(s)]
    table = (src, [d] * s, [1] * s, s, n, d, r, query.data_ptr(), 1, 2**-23, 0.5)
    _native.forward(*table, out.data_ptr(), d, logits.data_ptr(), stats.data_ptr(), 0, stream)
    want = torch.empty_like(values)
    got = torch.full_like(values, float("nan"))
    _native.backward(*table, upstream.data_ptr(), d, 1, logits.data_ptr(), stats.data_ptr(),
                     [want.data_ptr() + i * step for i in range(s)], [d] * s, None, 0, None, None,
                     0, stream)
    status = _native.backward_static_scratch(
        *table, upstream.data_ptr(), d, 1, logits.data_ptr(), stats.data_ptr(),
        [got.data_ptr() + i * step for i in range(s)], [d] * s, None, None, 0, stream)
    torch.cuda.synchronize()
    assert status == 0, _native.status_text(status)
    assert torch.equal(got, want)
