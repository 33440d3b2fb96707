"""Backward that accumulates value gradients into caller-owned buffers (C-ABI flag
ATTNRES_B200_FLAG_ACCUMULATE_DV, Python `attnres.accumulate.attnres_accumulate`).

Oracle: the sum over reads of the oracle's per-read value gradients, formed in FP32 and
rounded to BF16 once; tolerance rtol = atol = 0.05 as for every gradient of the path
(validation/protocol.json:12-15 of the reference)."""
import pytest
import torch

from oracle import attnres_oracle as ao

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
TOL = dict(rtol=0.05, atol=0.05)

SHAPES = [
    (9, 700, 2048, 2048),     # one-pass kernel, two-warp groups, several positions per group
    (49, 500, 4096, 4096),    # four-warp groups, odd source count
    (6, 1500, 1024, 1024),    # one-warp groups, even source count
    (1, 600, 1024, 1024), (2, 600, 2048, 512),
    (16, 300, 4096, 1024),    # low-rank tail
    (5, 200, 8192, 8192),     # eight-warp groups
    (7, 333, 1536, 128),      # partial last lane group
    (3, 11, 200, 72), (5, 9, 3000, 257),   # generic kernel
]


@pytest.mark.parametrize("as_list", [False, True], ids=["packed", "list"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_three_reads_accumulate_into_the_buffers(shape, as_list):
    from attnres import attnres
    from attnres.accumulate import attnres_accumulate
    torch.manual_seed(20261125)
    s, n, d, r = shape
    values = torch.randn(s, n, d, device="cuda", dtype=BF16)
    queries = [(torch.randn(r, device="cuda", dtype=BF16) * 0.1).requires_grad_() for _ in range(3)]
    upstreams = [torch.randn(n, d, device="cuda", dtype=BF16) for _ in range(3)]
    scale = r ** -0.5 if r != d else 1.0
    start = torch.randn(s, n, d, device="cuda", dtype=BF16)     # the buffers do not start at zero

    packed_buffer = start.clone()
    buffers = packed_buffer if not as_list else [packed_buffer[i] for i in range(s)]
    arg = values if not as_list else tuple(values.unbind(0))
    expected = start.float()
    peak = expected.abs()
    for query, upstream in zip(queries, upstreams):
        out = attnres_accumulate(arg, query, buffers, scale=scale)
        plain = attnres(arg, query.detach(), scale=scale)
        assert torch.equal(out, plain)
        out.backward(upstream)
        e_out, e_dv, e_dq = ao.oracle_with_grads(values, query.detach(), upstream, scale=scale)
        torch.testing.assert_close(out.detach(), e_out, **TOL)
        torch.testing.assert_close(query.grad, e_dq, **TOL)
        expected += e_dv.float()
        peak = torch.maximum(peak, expected.abs())
    # The buffer is BF16: each of the three additions rounds at the magnitude the running sum
    # has at that moment (half an ulp = 2^-9 relative), which can exceed the final value's
    # own tolerance where the contributions cancel.
    allowed = 0.05 + 0.05 * expected.abs() + 3 * 2.0**-9 * peak
    excess = ((packed_buffer.float() - expected).abs() - allowed).max().item()
    assert excess <= 0, excess
    error = (packed_buffer.float() - expected).norm() / expected.norm()
    assert error < 1e-2, error


def test_accumulation_is_more_exact_than_summing_rounded_gradients():
    """dsrc += dV adds the FP32 gradient and rounds once; autograd's accumulation rounds the
    gradient first and the sum again."""
    from attnres import attnres
    from attnres.accumulate import attnres_accumulate
    torch.manual_seed(5)
    s, n, d = 8, 256, 2048
    values = torch.randn(s, n, d, device="cuda", dtype=BF16, requires_grad=True)
    buffer = torch.zeros(s, n, d, device="cuda", dtype=BF16)
    exact = torch.zeros(s, n, d, device="cuda", dtype=torch.float32)
    rounded = torch.zeros(s, n, d, device="cuda", dtype=BF16)
    for _ in range(6):
        query = (torch.randn(d, device="cuda", dtype=BF16) * 0.05).requires_grad_()
        upstream = torch.randn(n, d, device="cuda", dtype=BF16)
        attnres_accumulate(values.detach(), query, buffer).backward(upstream)
        dv, = torch.autograd.grad(attnres(values, query), (values,), upstream)
        rounded += dv
        exact += ao.oracle_with_grads(values, query.detach(), upstream)[1].float()
    fused_error = (buffer.float() - exact).norm()
    autograd_error = (rounded.float() - exact).norm()
    assert fused_error <= autograd_error * 1.02, (fused_error, autograd_error)


def test_sources_receive_no_autograd_gradient_and_query_may_be_constant():
    from attnres.accumulate import attnres_accumulate
    torch.manual_seed(1)
    sources = [torch.randn(40, 1024, device="cuda", dtype=BF16, requires_grad=True) for _ in range(3)]
    buffers = [torch.zeros(40, 1024, device="cuda", dtype=BF16) for _ in range(3)]
    query = torch.randn(1024, device="cuda", dtype=BF16) * 0.1          # no grad wanted
    out = attnres_accumulate(sources, query, buffers)
    out.backward(torch.ones_like(out))
    assert all(source.grad is None for source in sources)
    assert all(bool(buffer.float().abs().sum() > 0) for buffer in buffers)


def test_c_abi_accumulate_flag_needs_gradient_rows():
    from attnres import _native
    lib = _native.load()
    ptrs = _native.pointer_array([0x1000] * 2)
    strides = _native.int64_array([16] * 2)
    ones = _native.int64_array([1] * 2)
    status = lib.attnres_b200_backward(ptrs, strides, ones, 2, 4, 16, 8, 0x2000, 1, 2**-23, 1.0,
                                       0x6000, 16, 1, 0x4000, 0x5000, None, None, None, None,
                                       0x7000, 4, 0x8000, None, _native.FLAG_ACCUMULATE_DV, None)
    assert status == 1


@pytest.mark.parametrize("shape", [(9, 400, 2048, 2048), (3, 200, 1024, 256), (5, 9, 3000, 257)],
                         ids=lambda s: "x".join(map(str, s)))
def test_overwrite_makes_the_first_read_store_instead_of_add(shape):
    """`overwrite=True` for the read whose backward runs first: no zeroing of the buffers."""
    from attnres.accumulate import attnres_accumulate
    torch.manual_seed(3)
    s, n, d, r = shape
    values = torch.randn(s, n, d, device="cuda", dtype=BF16)
    buffers = [torch.full((n, d), float("nan"), device="cuda", dtype=BF16) for _ in range(s)]
    expected = torch.zeros(s, n, d, device="cuda", dtype=torch.float32)
    for index in range(2):
        query = (torch.randn(r, device="cuda", dtype=BF16) * 0.1).requires_grad_()
        upstream = torch.randn(n, d, device="cuda", dtype=BF16)
        out = attnres_accumulate(tuple(values.unbind(0)), query, buffers, scale=r ** -0.5,
                                 overwrite=index == 0)
        out.backward(upstream)
        expected += ao.oracle_with_grads(values, query.detach(), upstream, scale=r ** -0.5)[1].float()
    torch.testing.assert_close(torch.stack(buffers).float(), expected, **TOL)


@pytest.mark.parametrize("shape", [(6, 130, 2048, 2048), (4, 50, 264, 72)],
                         ids=lambda s: "x".join(map(str, s)))
def test_accumulate_reads_strided_sources_and_stays_inside_its_buffers(shape):
    """Sources that are column slices of wider producers (row stride > D) and gradient buffers
    carved out of one poisoned allocation: the bands between and around them stay untouched."""
    from attnres.accumulate import attnres_accumulate
    torch.manual_seed(9)
    s, n, d, r = shape
    producers = [torch.randn(n, d + 8, device="cuda", dtype=BF16) for _ in range(s)]
    sources = [p[:, :d] for p in producers]
    pad = 128
    whole = torch.full((s * (n * d + pad) + pad,), -3.0, device="cuda", dtype=BF16)
    buffers = [whole[pad + i * (n * d + pad): pad + i * (n * d + pad) + n * d].view(n, d)
               for i in range(s)]
    for buffer in buffers:
        buffer.zero_()
    query = (torch.randn(r, device="cuda", dtype=BF16) * 0.1).requires_grad_()
    upstream = torch.randn(n, d, device="cuda", dtype=BF16)
    attnres_accumulate(sources, query, buffers, scale=0.25).backward(upstream)
    values = torch.stack([x.contiguous() for x in sources])
    _, e_dv, e_dq = ao.oracle_with_grads(values, query.detach(), upstream, scale=0.25)
    torch.testing.assert_close(torch.stack(buffers), e_dv, **TOL)
    torch.testing.assert_close(query.grad, e_dq, **TOL)
    for i in range(s + 1):
        band = whole[i * (n * d + pad): i * (n * d + pad) + pad]
        assert bool((band == -3.0).all()), f"band {i} was written"


def test_accumulating_and_sharded_reads_trace_under_torch_compile():
    """Both extensions are torch.library operators (the accumulating backward declares its
    buffers as mutated arguments): one full graph, no graph break, same bits as eager."""
    from attnres.accumulate import attnres_accumulate
    from attnres.parallel import sharded_attnres
    torch.manual_seed(9)
    s, n, d = 6, 300, 1024
    sources = [torch.randn(n, d, device="cuda", dtype=BF16) for _ in range(s)]
    upstream = torch.randn(n, d, device="cuda", dtype=BF16)

    def accumulate_step(query, buffers):
        out = attnres_accumulate(sources, query, buffers)
        return (out.float() * upstream.float()).sum()

    def sharded_step(query, leaves):
        out = sharded_attnres(leaves, query)        # no process group: the local read
        return (out.float() * upstream.float()).sum()

    query = (torch.randn(d, device="cuda", dtype=BF16) * 0.1).requires_grad_()
    eager_buffers = [torch.ones(n, d, device="cuda", dtype=BF16) for _ in range(s)]
    accumulate_step(query, eager_buffers).backward()
    eager_dq = query.grad.clone()

    before = torch._dynamo.utils.counters["stats"]["unique_graphs"]
    query2 = query.detach().clone().requires_grad_()
    compiled_buffers = [torch.ones(n, d, device="cuda", dtype=BF16) for _ in range(s)]
    torch.compile(accumulate_step, fullgraph=True, dynamic=False)(query2, compiled_buffers).backward()
    assert torch.equal(query2.grad, eager_dq)
    for a, e in zip(compiled_buffers, eager_buffers):
        assert torch.equal(a, e)
    assert torch._dynamo.utils.counters["stats"]["unique_graphs"] - before == 1

    leaves = [t.clone().requires_grad_() for t in sources]
    query3 = query.detach().clone().requires_grad_()
    sharded_step(query3, leaves).backward()
    leaves2 = [t.clone().requires_grad_() for t in sources]
    query4 = query.detach().clone().requires_grad_()
    torch.compile(sharded_step, fullgraph=True, dynamic=False)(query4, leaves2).backward()
    assert torch.equal(query4.grad, query3.grad)
    for a, e in zip(leaves2, leaves):
        assert torch.equal(a.grad, e.grad)
    # with a single rank the sharded read is the plain read
    from attnres import attnres
    query5 = query.detach().clone().requires_grad_()
    (attnres(sources, query5).float() * upstream.float()).sum().backward()
    assert torch.equal(query5.grad, query3.grad)
