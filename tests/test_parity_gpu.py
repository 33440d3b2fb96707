"""GPU parity of the CUDA kernels (through the C ABI) against the oracle.

Tolerance: the reference's protocol, rtol = atol = 0.05 on BF16 outputs, value
gradients and query gradients (validation/protocol.json:12-15), plus tighter
relative-L2 bounds stated per test.  Shapes are the reference's envelope
(validation/protocol.json:16-112, tests/test_cuda.py:27-31, :296-305 and
tests/test_bf16_packed_kernels.py of the reference) and the shapes of its benchmark configurations.
"""
import gc
import weakref
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attnres_oracle as ao

pytestmark = pytest.mark.gpu

TOL = dict(rtol=0.05, atol=0.05)
GOLDEN = np.load(Path(__file__).parent / "golden" / "reference_oracle.npz")
BF16 = torch.bfloat16


@pytest.fixture(params=["auto", "generic", "stream"])
def family(request):
    """Run a test with the library's own kernel choice, forced onto the layout-generic
    kernels, and with the forward saving its output residual for the one-pass backward
    wherever that kernel supports the shape (elsewhere the residual is written and unused)."""
    from attnres import _native, _ops
    flags = {"auto": 0, "generic": _native.FLAG_FORCE_GENERIC,
             "stream": _native.FLAG_PREFER_STREAM}[request.param]
    previous = _ops.set_kernel_flags(flags)
    yield request.param
    _ops.set_kernel_flags(previous)


def _close(actual, expected, what=""):
    assert actual.dtype == BF16, what
    assert torch.isfinite(actual).all() and torch.isfinite(expected).all(), what
    torch.testing.assert_close(actual, expected, **TOL, msg=lambda m: f"{what}: {m}")
    return ao.error_metrics(actual, expected)


def _check_triplet(actual, expected, l2_bound=2e-2):
    names = ("out", "dvalues", "dquery")
    for name, a, e in zip(names, actual, expected):
        metrics = _close(a, e, name)
        assert metrics["relative_l2"] < l2_bound, (name, metrics)


def _single(shape, *, strided=True, scale=1.0, eps=2**-23, zero_query=False, as_list=False,
            query_std=0.25):
    """One call on a strided producer with a transposed upstream
    (validation/gpu_checks.py:30-47 of the reference)."""
    from attnres import attnres
    s, n, d, r = shape
    producer = torch.randn(s, n, d + (7 if strided else 0), device="cuda", dtype=BF16,
                           requires_grad=True)
    query = (torch.zeros(r, device="cuda", dtype=BF16) if zero_query
             else torch.randn(r, device="cuda", dtype=BF16) * query_std).requires_grad_()
    values = producer[..., :d]
    arg = tuple(values.unbind(0)) if as_list else values
    actual = attnres(arg, query, eps=eps, scale=scale)
    expected = ao.oracle(values, query, eps=eps, scale=scale)
    upstream = torch.randn(d, n, device="cuda", dtype=BF16).transpose(0, 1)
    ga = torch.autograd.grad(actual, (producer, query), upstream)
    ge = torch.autograd.grad(expected, (producer, query), upstream)
    _check_triplet((actual, *ga), (expected, *ge))


# ------------------------------------------------------------------ golden vectors

@pytest.mark.parametrize("name", [str(n) for n in GOLDEN["names"]])
def test_golden_vectors(name, family):
    from attnres import attnres
    get = lambda key: ao.from_bf16_bits(GOLDEN[f"{name}.{key}"]).cuda()
    eps, scale = (float(x) for x in GOLDEN[f"{name}.eps_scale"])
    values, query = get("values").requires_grad_(), get("query").requires_grad_()
    for arg in (values, tuple(values.unbind(0))):
        out = attnres(arg, query, eps=eps, scale=scale)
        dv, dq = torch.autograd.grad(out, (values, query), get("upstream"))
        _check_triplet((out, dv, dq), (get("out"), get("dv"), get("dq")), l2_bound=1e-2)


# ------------------------------------------------------------------ envelope

ENVELOPE = [
    (1, 1, 1, 1), (1, 2, 128, 16), (9, 65, 768, 64), (33, 128, 1536, 128), (97, 16, 4096, 64),
    (129, 8, 7168, 128), (129, 8, 8192, 8192), (9, 32, 3000, 127),            # protocol smoke
    (13, 67, 512, 3), (73, 129, 2048, 64), (127, 31, 5120, 256), (17, 257, 6144, 127),  # held out
    (5, 7, 3000, 257), (129, 1, 8192, 6144), (3, 2, 17, 5), (2, 3, 8, 8), (4, 5, 24, 16),
    (9, 19, 1024, 1023), (33, 17, 1536, 769), (33, 19, 2047, 1024), (9, 65, 2049, 1025),
]


@pytest.mark.parametrize("as_list", [False, True], ids=["packed", "list"])
@pytest.mark.parametrize("shape", ENVELOPE, ids=lambda s: "x".join(map(str, s)))
def test_envelope_strided_producer(shape, as_list, family):
    torch.manual_seed(20260827)
    _single(shape, strided=True, as_list=as_list)


@pytest.mark.parametrize("as_list", [False, True], ids=["packed", "list"])
@pytest.mark.parametrize("shape", ENVELOPE, ids=lambda s: "x".join(map(str, s)))
def test_envelope_contiguous(shape, as_list, family):
    torch.manual_seed(20260903)
    _single(shape, strided=False, as_list=as_list)


def test_zero_query_with_negative_scale(family):
    torch.manual_seed(20260827)
    _single((2, 11, 128, 16), scale=-0.5, zero_query=True)


@pytest.mark.parametrize("eps,scale", [(2**-20, 0.75), (2**-10, -0.75), (1e-3, 0.0)])
def test_eps_and_scale_reach_the_kernels(eps, scale, family):
    torch.manual_seed(5)
    _single((5, 9, 264, 72), eps=eps, scale=scale, strided=False)


# ------------------------------------------------------------------ benchmark shapes (reduced rows)

SWEEP = [(s, d) for d in (1024, 2048, 4096) for s in (2, 5, 9, 17, 25, 49)]


@pytest.mark.parametrize("as_list", [False, True], ids=["packed", "list"])
@pytest.mark.parametrize("sources,width", SWEEP)
def test_operator_sweep_shapes_reduced_rows(sources, width, as_list, family):
    """The operator sweep (benchmark configuration 2) at N = 384 rows: values ~N(0,1), query
    ~N(0,0.02), R = D."""
    torch.manual_seed(20260827 + sources + width)
    _single((sources, 384, width, width), strided=False, as_list=as_list, query_std=0.02)


@pytest.mark.parametrize("rank,scale", [(1024, 1 / 32), (4096, 1 / 64)])
def test_sliced_low_rank_shape_reduced_rows(rank, scale, family):
    """The sliced low-rank shape (benchmark configuration 3) at N = 512 rows: S = 16, D = 4096,
    R = 1024 (and R = D)."""
    torch.manual_seed(20260903)
    _single((16, 512, 4096, rank), strided=False, scale=scale, query_std=0.02)


@pytest.mark.parametrize("sources", [2, 4, 7])
def test_block_schedule_shape_reduced_rows(sources, family):
    """The reads of the D = 4096 Block-schedule model (benchmark configuration 5): R = 1024,
    S <= 7."""
    torch.manual_seed(20260911)
    _single((sources, 300, 4096, 1024), strided=False, as_list=True, scale=1 / 32, query_std=0.02)


# ------------------------------------------------------------------ full-size shapes

@pytest.mark.parametrize("sources,width,rank", [(9, 2048, 2048), (2, 1024, 1024), (17, 4096, 4096),
                                                (16, 4096, 1024),
                                                # cells of the sweep served by the staged two-pass kernel
                                                (9, 1024, 1024), (25, 1024, 1024), (25, 2048, 2048)])
def test_full_size_rows_against_oracle_and_row_independence(sources, width, rank):
    """N = 16 384 rows (benchmark configurations 2 and 3).  Checks (a) parity with the oracle
    evaluated on the device, (b) positions are independent: any row block computed alone
    gives the same bits as inside the full call, (c) the output is a convex combination
    of the sources, (d) the query gradient of the whole equals the sum over row blocks."""
    from attnres import attnres
    torch.manual_seed(20260827)
    n = 16384
    values = torch.randn(sources, n, width, device="cuda", dtype=BF16).requires_grad_()
    query = (torch.randn(rank, device="cuda", dtype=BF16) * 0.02).requires_grad_()
    upstream = torch.randn(n, width, device="cuda", dtype=BF16)
    scale = rank ** -0.5 if rank != width else 1.0
    out = attnres(values, query, scale=scale)
    dv, dq = torch.autograd.grad(out, (values, query), upstream)
    expected = ao.oracle(values, query, scale=scale)
    ev, eq = torch.autograd.grad(expected, (values, query), upstream)
    _check_triplet((out, dv, dq), (expected, ev, eq), l2_bound=1e-2)
    del expected, ev
    # (c) convexity, up to one BF16 rounding of the result
    low, high = values.detach().amin(0).float(), values.detach().amax(0).float()
    slack = out.float().abs() * 2**-8 + 1e-6
    assert bool(((out.float() >= low - slack) & (out.float() <= high + slack)).all())
    # (b) + (d)
    total = torch.zeros(rank, device="cuda", dtype=torch.float32)
    for start, stop in ((0, 1), (1, 4097), (4097, 12000), (12000, n)):
        block = values.detach()[:, start:stop].clone().requires_grad_()
        q2 = query.detach().clone().requires_grad_()
        o2 = attnres(block, q2, scale=scale)
        dv2, dq2 = torch.autograd.grad(o2, (block, q2), upstream[start:stop])
        assert torch.equal(o2, out[start:stop])
        assert torch.equal(dv2, dv[:, start:stop])
        total += dq2.float()
    torch.testing.assert_close(total, dq.float(), rtol=0.02, atol=0.02 * float(dq.float().abs().max()))


# ------------------------------------------------------------------ layouts

def _mixed_layout_case(shape, *, shared=False):
    """Sources with three physical layouts (feature-strided, transposed, padded), a strided
    query and a transposed upstream (validation/source_checks.py:40-92 of the reference)."""
    from attnres import attnres
    s, n, d, r = shape
    count = s - 1 if shared and s > 1 else s
    leaves = [torch.randn(*((n, 2 * d), (d, n), (n, d + 7))[i % 3], device="cuda", dtype=BF16,
                          requires_grad=True) for i in range(count)]
    query = torch.randn(2 * r, device="cuda", dtype=BF16, requires_grad=True)
    upstream = torch.randn(d, n, device="cuda", dtype=BF16).T

    def views():
        rows = [a[..., ::2] if i % 3 == 0 else a.T if i % 3 == 1 else a[..., :d]
                for i, a in enumerate(leaves)]
        if shared and s > 1:
            rows.append(rows[0])
        return tuple(rows)

    params = (*leaves, query)
    for packed in (False, True):
        arg = torch.stack(views()) if packed else views()
        actual = attnres(arg, query[::2])
        ga = torch.autograd.grad(actual, params, upstream, retain_graph=True)
        repeat = torch.autograd.grad(actual, params, upstream)
        for a, b in zip(ga, repeat):
            assert torch.equal(a, b), "backward is not bit-reproducible"
        expected = ao.oracle(torch.stack(views()) if packed else views(), query[::2])
        ge = torch.autograd.grad(expected, params, upstream)
        _close(actual, expected, "out")
        for a, e in zip(ga, ge):
            _close(a, e, "grad")


@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (5, 7, 128, 128), (5, 7, 128, 16), (9, 19, 1024, 32),
                                   (33, 7, 2047, 257), (7, 9, 513, 257), (129, 8, 7168, 1024),
                                   (129, 7, 2048, 2048)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("shared", [False, True])
def test_source_lists_with_mixed_physical_layouts(shape, shared, family):
    torch.manual_seed(20260827)
    _mixed_layout_case(shape, shared=shared)


def test_feature_and_query_strides_packed(family):
    # tests/test_cuda.py:34-54 of the reference
    from attnres import attnres
    torch.manual_seed(20260827)
    s, n, d, r = 9, 7, 1536, 769
    values = torch.randn(s, n, 2 * d, device="cuda", dtype=BF16, requires_grad=True)
    query = (torch.randn(2 * r, device="cuda", dtype=BF16) * 0.25).requires_grad_()
    upstream = torch.randn(d, n, device="cuda", dtype=BF16).T
    actual = attnres(values[..., ::2], query[::2])
    expected = ao.oracle(values[..., ::2], query[::2])
    ga = torch.autograd.grad(actual, (values, query), upstream)
    ge = torch.autograd.grad(expected, (values, query), upstream)
    _check_triplet((actual, *ga), (expected, *ge))


@pytest.mark.parametrize("rank", [17, 5])
@pytest.mark.parametrize("as_list", [False, True])
@pytest.mark.parametrize("swap", ["upstream", "sources"])
def test_non_affine_batches(rank, as_list, swap, family):
    """Batch axes that cannot be flattened to one row stride, on the upstream gradient
    (tests/test_cuda.py:272-293 of the reference) or on the sources themselves."""
    from attnres import attnres
    torch.manual_seed(20260827)
    values = torch.randn(3, 2, 3, 17, device="cuda", dtype=BF16, requires_grad=True)
    query = torch.randn(rank, device="cuda", dtype=BF16, requires_grad=True)
    if swap == "upstream":
        base = values                                                          # sources [2,3,17]
        upstream = torch.randn(3, 2, 17, device="cuda", dtype=BF16).transpose(0, 1)
    else:
        base = values.transpose(1, 2)                                          # sources [3,2,17]
        upstream = torch.randn(3, 2, 17, device="cuda", dtype=BF16)
    arg = tuple(base.unbind(0)) if as_list else base
    actual = attnres(arg, query)
    expected = ao.oracle(base, query)
    ga = torch.autograd.grad(actual, (values, query), upstream)
    ge = torch.autograd.grad(expected, (values, query), upstream)
    _check_triplet((actual, *ga), (expected, *ge))


@pytest.mark.parametrize("layout", ["singleton", "nonaffine"])
@pytest.mark.parametrize("sources", [2, 4])
def test_storage_offset_and_shared_leaves(layout, sources, family):
    """Leaves start one element into their storage (2-byte-aligned base), one source is
    used twice, query has stride 2 (validation/layout_checks.py:15-70 of the reference)."""
    from attnres import attnres
    torch.manual_seed(20260827)
    width, rank = 32, 16
    rows = 3 if layout == "singleton" else 6
    leaves = tuple(torch.randn(rows * width + 1, device="cuda", dtype=BF16, requires_grad=True)
                   for _ in range(sources - (sources == 4)))
    query = (torch.randn(rank * 2, device="cuda", dtype=BF16) * 0.05).requires_grad_()
    raw_upstream = torch.randn(rows * width, device="cuda", dtype=BF16)

    def view(value):
        if layout == "singleton":
            return value[1:].as_strided((3, 1, width), (width, 2 * width, 1))
        return value[1:].view(2, 3, width).transpose(0, 1)

    upstream = (raw_upstream.as_strided((3, 1, width), (width, 3 * width, 1))
                if layout == "singleton" else raw_upstream.view(2, 3, width).transpose(0, 1))

    def forward(op):
        values = tuple(view(value) for value in leaves)
        if sources == 4:
            values = (*values, values[1])
        return op(values, query[::2], eps=2**-10, scale=-0.75)

    actual = forward(attnres)
    ga = torch.autograd.grad(actual, (*leaves, query), upstream)
    expected = forward(ao.oracle)
    ge = torch.autograd.grad(expected, (*leaves, query), upstream)
    _close(actual, expected)
    for a, e in zip(ga, ge):
        _close(a, e)


def test_offsets_beyond_int32(family):
    """Source bases and row strides more than 2^31 elements apart
    (tests/test_offsets.py:13-59 of the reference)."""
    from attnres import attnres
    torch.manual_seed(20260827)
    stride = 2**31 + 32
    # packed: two sources 2^31+32 elements apart
    width, rank = 8192, 127
    storage = torch.empty(stride + width, device="cuda", dtype=BF16)
    values = storage.as_strided((2, 1, width), (stride, width, 1)).detach()
    values.copy_(torch.randn_like(values))
    values.requires_grad_()
    query = (torch.randn(rank, device="cuda", dtype=BF16) * 0.25).requires_grad_()
    actual = attnres(values, query)
    expected = ao.oracle(values, query)
    upstream = torch.randn_like(actual)
    ga = torch.autograd.grad(actual, (values, query), upstream)
    ge = torch.autograd.grad(expected, (values, query), upstream)
    _check_triplet((actual, *ga), (expected, *ge))
    del values, ga, ge, actual, expected
    # list: one source whose ROW stride exceeds 2^31
    for width, rank in ((17, 17), (17, 5), (64, 64)):
        value = storage.as_strided((2, width), (stride, 1)).detach()
        value.copy_(torch.randn_like(value))
        value.requires_grad_()
        other = torch.randn(2, width, device="cuda", dtype=BF16, requires_grad=True)
        query = (torch.randn(rank, device="cuda", dtype=BF16) * 0.25).requires_grad_()
        actual = attnres((value, other), query)
        expected = ao.oracle(torch.stack((value, other)), query)
        upstream = torch.randn_like(actual)
        ga = torch.autograd.grad(actual, (value, other, query), upstream)
        ge = torch.autograd.grad(expected, (value, other, query), upstream)
        _close(actual, expected)
        for a, e in zip(ga, ge):
            _close(a, e)


def test_overlapping_views_keep_distinct_gradients(family):
    # tests/test_cuda.py:149-172 of the reference
    from attnres import attnres
    torch.manual_seed(20260827)
    shared = torch.randn(5, 18, device="cuda", dtype=BF16)
    values = (shared[:, :17].detach().requires_grad_(), shared[:, 1:].detach().requires_grad_(),
              torch.randn(5, 17, device="cuda", dtype=BF16, requires_grad=True))
    query = torch.randn(5, device="cuda", dtype=BF16, requires_grad=True)
    actual = attnres(values, query)
    expected = ao.oracle(torch.stack(values), query)
    upstream = torch.randn_like(actual)
    ga = torch.autograd.grad(actual, (*values, query), upstream)
    ge = torch.autograd.grad(expected, (*values, query), upstream)
    assert not torch.equal(ge[0], ge[1])
    _close(actual, expected)
    for a, e in zip(ga, ge):
        _close(a, e)


# ------------------------------------------------------------------ exact regimes

@pytest.mark.parametrize("sources,rows,packed", [(2, 2, False), (4, 2, False), (4, 2, True),
                                                 (4, 1024, False), (8, 64, True)])
@pytest.mark.parametrize("scale", [2.0**24, -(2.0**24)])
@pytest.mark.parametrize("width,rank", [(256, 16), (1024, 1024)])
def test_equal_logits_are_exact_and_survive_graph_replay(sources, rows, packed, scale, width, rank,
                                                         family):
    """All-ones sources at |logit| ~ 2.7e8: output == source, dV == dO/S, dq == 0, exactly,
    eagerly and in CUDA-graph replays with a changed upstream
    (validation/softmax_checks.py:9-50 of the reference)."""
    from attnres import attnres
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        values = torch.ones(sources, rows, width, device="cuda", dtype=BF16, requires_grad=True)
        query = torch.ones(rank, device="cuda", dtype=BF16, requires_grad=True)
        inputs = values if packed else tuple(values.unbind())
        upstream = torch.ones_like(values[0])

        def call():
            out = attnres(inputs, query, eps=2**-23, scale=scale)
            return (out, *torch.autograd.grad(out, (values, query), upstream))

        def check(result):
            out, dv, dq = result
            assert torch.equal(out, values[0])
            assert torch.equal(dv, upstream.expand_as(values) / sources)
            assert torch.equal(dq, torch.zeros_like(query))

        check(call())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            result = call()
        for factor in (-2.0, 4.0):
            upstream.fill_(factor)
            graph.replay()
            torch.cuda.synchronize()
            check(result)
    torch.cuda.current_stream().wait_stream(stream)


def _fill_routing(values, query, upstream, kind, iteration):
    """Numeric regimes of validation/routing_checks.py:11-37 of the reference."""
    sources, _, _ = values.shape
    rank = query.numel()
    with torch.no_grad():
        values.normal_()
        query.normal_(std=0.05)
        upstream.normal_()
        values[..., :-rank].add_(torch.arange(sources, device=values.device)[:, None, None])
        if kind in ("zero_keys", "tiny_keys"):
            values[..., -rank:].mul_(0 if kind == "zero_keys" else 2**-12)
            return 2**-10, -0.75
        if kind == "zero_scale":
            return 2**-10, 0.0
        if kind == "large_logits":
            values[..., -rank:].zero_()
            values[..., -rank] = 1
            values[..., -rank + 1] = torch.tensor(
                [1.0 if (s + iteration) % 2 else -1.0 for s in range(sources)],
                device=values.device)[:, None]
            query.zero_()
            query[0] = 1 + iteration / 8
            query[1] = 2**-22
            return 2**-10, 2.0**20
        return 2**-10, -0.75


@pytest.mark.parametrize("kind", ["zero_keys", "tiny_keys", "zero_scale", "large_logits",
                                  "negative_scale"])
@pytest.mark.parametrize("rows,width,rank", [(7, 64, 16), (33, 1024, 256), (5, 520, 520)])
def test_routing_regimes_with_graph_replay(kind, rows, width, rank, family):
    from attnres import attnres
    torch.manual_seed(20260906)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        values = torch.empty(4, rows, width, device="cuda", dtype=BF16, requires_grad=True)
        query = torch.empty(rank, device="cuda", dtype=BF16, requires_grad=True)
        upstream = torch.empty(width, rows, device="cuda", dtype=BF16).T
        eps, scale = _fill_routing(values, query, upstream, kind, 0)

        def call():
            out = attnres(tuple(values.unbind()), query, eps=eps, scale=scale)
            return (out, *torch.autograd.grad(out, (values, query), upstream))

        def check(actual):
            if kind == "large_logits":
                # |z| ~ 3e6: one FP32 ulp of a logit is 0.25, so two correct evaluations of z
                # (the oracle normalises then dots, the kernels dot then scale, as the
                # reference's list kernel does, src/attnres/_kernels/fla_full_sources.py:389-394)
                # give visibly different weights.  Hold the kernel's saved logits to 4 ulp of
                # the float64 value and everything downstream to the closed form GIVEN them.
                _, logits, _, _ = torch.ops.attnres_b200.read_sources_forward(
                    list(values.detach().unbind()), query.detach(), float(eps), float(scale))
                v64 = values.detach().double().cpu().numpy()
                q64 = query.detach().double().cpu().numpy()
                g64 = upstream.double().cpu().numpy()
                tail = v64[..., -rank:]
                exact = scale * (tail * q64).sum(-1) / np.sqrt((tail * tail).mean(-1) + eps)
                np.testing.assert_allclose(logits.double().cpu().numpy(), exact, rtol=4 * 2**-23)
                expected = ao.closed_form(v64, q64, g64, eps=eps, scale=scale,
                                          logits=logits.double().cpu().numpy())
                for a, e in zip(actual[:2], expected[:2]):
                    _close(a, torch.from_numpy(e).to(BF16).to(a.device), kind)
                # dquery sums +-1e6-sized terms that cancel to O(1): hold it to the closed
                # form within four times the error the FP32 oracle itself makes there.
                truth = ao.closed_form(v64, q64, g64, eps=eps, scale=scale)[2]
                reference = ao.oracle(tuple(values.unbind()), query, eps=eps, scale=scale)
                _, oracle_dq = torch.autograd.grad(reference, (values, query), upstream)
                oracle_error = np.abs(oracle_dq.double().cpu().numpy() - truth).max()
                ours_error = np.abs(actual[2].double().cpu().numpy() - expected[2]).max()
                assert ours_error <= max(0.05, 4.0 * oracle_error), (ours_error, oracle_error)
                return
            expected = ao.oracle(tuple(values.unbind()), query, eps=eps, scale=scale)
            ge = torch.autograd.grad(expected, (values, query), upstream)
            for a, e in zip(actual, (expected, *ge)):
                _close(a, e, kind)
            if kind == "zero_keys":
                assert torch.equal(actual[2], torch.zeros_like(query))
            if kind == "zero_scale":
                assert torch.equal(actual[1], (upstream.expand_as(values) / 4).to(BF16))
                assert torch.equal(actual[2], torch.zeros_like(query))

        check(call())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = call()
        for iteration in range(1, 5):
            _fill_routing(values, query, upstream, kind, iteration)
            graph.replay()
            torch.cuda.synchronize()
            check(captured)
    torch.cuda.current_stream().wait_stream(stream)


# ------------------------------------------------------------------ autograd contract

def test_gradients_are_bit_reproducible_and_optional(family):
    from attnres import attnres
    torch.manual_seed(3)
    values = torch.randn(6, 333, 1024, device="cuda", dtype=BF16, requires_grad=True)
    query = torch.randn(1024, device="cuda", dtype=BF16, requires_grad=True)
    upstream = torch.randn(333, 1024, device="cuda", dtype=BF16)
    out = attnres(values, query)
    first = torch.autograd.grad(out, (values, query), upstream, retain_graph=True)
    second = torch.autograd.grad(out, (values, query), upstream, retain_graph=True)
    for a, b in zip(first, second):
        assert torch.equal(a, b)
    only_values, = torch.autograd.grad(out, (values,), upstream, retain_graph=True)
    only_query, = torch.autograd.grad(out, (query,), upstream, retain_graph=True)
    assert torch.equal(only_values, first[0]) and torch.equal(only_query, first[1])
    # a value-free graph: query only
    out2 = attnres(values.detach(), query)
    dq, = torch.autograd.grad(out2, (query,), upstream)
    assert torch.equal(dq, first[1])


def test_inputs_are_released_after_backward(family):
    # tests/test_cuda.py:175-217 of the reference
    from attnres import attnres
    torch.manual_seed(20260827)
    for as_list in (False, True):
        values = [torch.randn(5, 17, device="cuda", dtype=BF16, requires_grad=True) for _ in range(3)]
        query = torch.randn(5, device="cuda", dtype=BF16, requires_grad=True)
        refs = [weakref.ref(t) for t in (*values, query)]
        arg = tuple(values) if as_list else torch.stack(values)
        loss = attnres(arg, query).square().sum()
        del values, query, arg
        gc.collect()
        loss.backward()
        del loss
        torch.cuda.synchronize()
        gc.collect()
        assert all(ref() is None for ref in refs)


def test_learned_query_module_on_device(family):
    from attnres import LearnedQuery, attnres
    torch.manual_seed(1)
    module = LearnedQuery(64).cuda().float()
    values = torch.randn(4, 9, 256, device="cuda", dtype=BF16)
    out = attnres(values, module(), scale=0.125)
    out.float().sum().backward()
    assert module.query.grad.dtype == torch.float32 and module.query.grad.shape == (64,)
    expected = ao.oracle(values, module.query.detach().to(BF16), scale=0.125)
    _close(out, expected)


# ------------------------------------------------------------------ torch.compile / CUDA graphs

@pytest.mark.parametrize("shape", [(9, 65, 256, 32), (9, 65, 1024, 512), (33, 19, 2047, 1024),
                                   (5, 48, 2048, 2048), (49, 40, 2048, 2048)],
                         ids=lambda s: "x".join(map(str, s)))
def test_compiled_fullgraph_and_raw_graph_replay(shape):
    """torch.compile(fullgraph=True, dynamic=False) forward+backward, then a raw CUDA graph
    of the eager ops replayed with 8 changed inputs (validation/gpu_checks.py:77-132)."""
    from attnres import attnres
    torch.manual_seed(20260827)
    s, n, d, r = shape
    source = torch.randn(s, n, d + 3, device="cuda", dtype=BF16, requires_grad=True)
    query = torch.randn(r, device="cuda", dtype=BF16, requires_grad=True)
    upstream = torch.randn(n, d, device="cuda", dtype=BF16)

    def forward(v, q):
        return attnres(v[..., :d], q)

    compiled = torch.compile(forward, fullgraph=True, dynamic=False)
    before = None
    for step in range(3):
        out = compiled(source, query)
        go = torch.autograd.grad(out, (source, query), upstream)
        if step == 0:
            before = dict(torch._dynamo.utils.counters["stats"])
        with torch.no_grad():
            source.copy_(torch.randn_like(source))
    assert dict(torch._dynamo.utils.counters["stats"]) == before, "changed inputs recompiled"
    out = compiled(source, query)
    go = torch.autograd.grad(out, (source, query), upstream)
    expected = ao.oracle(source[..., :d], query)
    ge = torch.autograd.grad(expected, (source, query), upstream)
    _check_triplet((out, *go), (expected, *ge))

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        source = source.detach().clone().requires_grad_()
        query = query.detach().clone().requires_grad_()
        upstream = upstream.clone()
        for _ in range(3):
            torch.autograd.grad(forward(source, query), (source, query), upstream)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        captured = forward(source, query)
        captured_grads = torch.autograd.grad(captured, (source, query), upstream)
    pressure = [torch.full((65536 + i,), 17 + i, device="cuda", dtype=torch.int64) for i in range(4)]
    for _ in range(8):
        with torch.no_grad():
            source.copy_(torch.randn_like(source))
            query.copy_(torch.randn_like(query))
            upstream.copy_(torch.randn_like(upstream))
        graph.replay()
        torch.cuda.synchronize()
        expected = ao.oracle(source[..., :d], query)
        ge = torch.autograd.grad(expected, (source, query), upstream)
        _check_triplet((captured, *captured_grads), (expected, *ge))
    for i, tensor in enumerate(pressure):
        assert bool((tensor == 17 + i).all()), "an unrelated allocation was overwritten"


class _NoSourceStack(torch.utils._python_dispatch.TorchDispatchMode):
    """Fails if anything stacks or concatenates the source list
    (the guard of validation/source_checks.py:11-37 of the reference)."""

    def __init__(self, count):
        super().__init__()
        self.count = count

    @classmethod
    def ignore_compile_internals(cls):
        return True

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        if func in (torch.ops.aten.stack.default, torch.ops.aten.cat.default) and args[0]:
            if len(args[0]) == self.count:
                raise AssertionError("the source list was materialised as one tensor")
        return func(*args, **(kwargs or {}))


def test_compiled_source_list_never_packs_and_does_not_recompile():
    from attnres import attnres
    torch.manual_seed(20260827)
    n, d, r = 34, 512, 128
    leaves = [torch.randn(n, d + (i % 2) * 8, device="cuda", dtype=BF16, requires_grad=True)
              for i in range(5)]
    query = torch.randn(r, device="cuda", dtype=BF16, requires_grad=True)
    upstream = torch.randn(n, d, device="cuda", dtype=BF16)

    def forward(args, q):
        return attnres(tuple(a[..., :d] for a in args), q, scale=0.1)

    compiled = torch.compile(forward, fullgraph=True, dynamic=False)
    graphs_before = torch._dynamo.utils.counters["stats"]["unique_graphs"]
    for function in (forward, compiled, compiled):
        with _NoSourceStack(len(leaves)):
            out = function(leaves, query)
            grads = torch.autograd.grad(out, (*leaves, query), upstream)
        expected = ao.oracle(tuple(a[..., :d] for a in leaves), query, scale=0.1)
        ge = torch.autograd.grad(expected, (*leaves, query), upstream)
        _close(out, expected)
        for a, e in zip(grads, ge):
            _close(a, e)
        with torch.no_grad():
            for leaf in leaves:
                leaf.copy_(torch.randn_like(leaf))
    assert torch._dynamo.utils.counters["stats"]["unique_graphs"] - graphs_before == 1


# ------------------------------------------------------------------ raw C ABI

@pytest.mark.parametrize("flags", [0, 1, 2])
@pytest.mark.parametrize("shape", [(5, 37, 1024, 1024), (3, 11, 200, 72), (4, 9, 2048, 512),
                                   (7, 21, 4096, 1024)])
def test_c_abi_direct_call_writes_only_its_outputs(shape, flags):
    """Calls the library with raw pointers.  Every output lives inside a larger poisoned
    buffer; the guard bands before and after it must be untouched."""
    from attnres import _native
    torch.manual_seed(7)
    s, n, d, r = shape
    dev = "cuda"
    values = torch.randn(s, n, d, device=dev, dtype=BF16)
    query = (torch.randn(r, device=dev, dtype=BF16) * 0.25)
    upstream = torch.randn(n, d, device=dev, dtype=BF16)
    pad = 256

    def guarded(numel, dtype):
        whole = torch.full((numel + 2 * pad,), -7, device=dev, dtype=dtype)
        return whole, whole[pad:pad + numel]

    out_w, out = guarded(n * d, BF16)
    logit_w, logits = guarded(s * n, torch.float32)
    stat_w, stats = guarded(2 * n, torch.float32)
    dv_w, dv = guarded(s * n * d, BF16)
    rows = _native.dq_workspace_rows(n, s, d, r, 0)
    part_w, partials = guarded(rows * r, torch.float32)
    dq_w, dq = guarded(r, BF16)
    dq32_w, dq32 = guarded(r, torch.float32)
    res_w, residual = guarded(n * d, torch.int16)
    saved = dict(out_ptr=out.data_ptr(), residual_ptr=residual.data_ptr()) if flags == 2 else {}
    stream = torch.cuda.current_stream().cuda_stream
    step = n * d * 2
    src = [values.data_ptr() + i * step for i in range(s)]
    _native.forward(src, [d] * s, [1] * s, s, n, d, r, query.data_ptr(), 1, 2**-23, 1.0,
                    out.data_ptr(), d, logits.data_ptr(), stats.data_ptr(), flags, stream,
                    residual_ptr=saved.get("residual_ptr"))
    _native.backward(src, [d] * s, [1] * s, s, n, d, r, query.data_ptr(), 1, 2**-23, 1.0,
                     upstream.data_ptr(), d, 1, logits.data_ptr(), stats.data_ptr(),
                     [dv.data_ptr() + i * step for i in range(s)], [d] * s,
                     partials.data_ptr(), rows, dq.data_ptr(), dq32.data_ptr(), flags, stream,
                     **saved)
    torch.cuda.synchronize()
    for whole in (out_w, logit_w, stat_w, dv_w, part_w, dq_w, dq32_w, res_w):
        assert bool((whole[:pad] == -7.0).all()) and bool((whole[-pad:] == -7.0).all())
    if flags != 2:
        assert bool((residual == -7.0).all()), "the residual was written without being asked for"
    e_out, e_dv, e_dq = ao.oracle_with_grads(values, query, upstream)
    _check_triplet((out.view(n, d), dv.view(s, n, d), dq), (e_out, e_dv, e_dq))
    # FP32 and BF16 forms of the query gradient agree, and the saved statistics are sane.
    assert torch.equal(dq32.to(BF16), dq)
    probs = torch.exp(logits.view(s, n) - stats[:n]) * stats[n:]
    torch.testing.assert_close(probs.sum(0), torch.ones(n, device=dev), rtol=1e-4, atol=1e-4)


# ------------------------------------------------------------------ one-pass backward

def _abi_forward_backward(values, query, upstream, *, flags, save, scale=1.0, eps=2**-23):
    """Forward + backward through the C ABI on contiguous inputs; returns
    (out, residual or None, dvalues, dquery FP32)."""
    from attnres import _native
    s, n, d = values.shape
    r = query.numel()
    out = torch.empty(n, d, device="cuda", dtype=BF16)
    residual = torch.empty(n, d, device="cuda", dtype=torch.int16) if save else None
    logits = torch.empty(s, n, device="cuda", dtype=torch.float32)
    stats = torch.empty(2, n, device="cuda", dtype=torch.float32)
    dv = torch.empty_like(values)
    rows = _native.dq_workspace_rows(n, s, d, r, 0)
    partials = torch.empty(rows, r, device="cuda", dtype=torch.float32)
    dq = torch.empty(r, device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    step = n * d * 2
    src = [values.data_ptr() + i * step for i in range(s)]
    _native.forward(src, [d] * s, [1] * s, s, n, d, r, query.data_ptr(), 1, eps, scale,
                    out.data_ptr(), d, logits.data_ptr(), stats.data_ptr(), flags, stream,
                    residual_ptr=residual.data_ptr() if save else None)
    _native.backward(src, [d] * s, [1] * s, s, n, d, r, query.data_ptr(), 1, eps, scale,
                     upstream.data_ptr(), d, 1, logits.data_ptr(), stats.data_ptr(),
                     [dv.data_ptr() + i * step for i in range(s)], [d] * s,
                     partials.data_ptr(), rows, None, dq.data_ptr(), flags, stream,
                     out_ptr=out.data_ptr() if save else None,
                     residual_ptr=residual.data_ptr() if save else None)
    torch.cuda.synchronize()
    return out, residual, dv, dq


@pytest.mark.parametrize("shape,flags", [((9, 300, 2048, 2048), 0), ((49, 200, 4096, 1024), 0),
                                         ((5, 33, 200, 72), 0), ((9, 300, 2048, 2048), 1)],
                         ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else str(v))
def test_output_residual_holds_what_the_rounding_dropped(shape, flags):
    """`out` joined with its 16-bit residual is the FP32 result: it rounds back to `out` bit
    for bit, matches the float64 closed form to FP32 accuracy, and asking for the residual
    does not change `out`."""
    torch.manual_seed(11)
    s, n, d, r = shape
    values = torch.randn(s, n, d, device="cuda", dtype=BF16)
    query = torch.randn(r, device="cuda", dtype=BF16) * 0.1
    upstream = torch.randn(n, d, device="cuda", dtype=BF16)
    out, residual, _, _ = _abi_forward_backward(values, query, upstream, flags=flags, save=True)
    plain, _, _, _ = _abi_forward_backward(values, query, upstream, flags=flags, save=False)
    assert torch.equal(out, plain)
    joined = ao.join_saved_output(out, residual)
    assert torch.isfinite(joined).all()
    assert torch.equal(joined.to(BF16), out)
    exact = ao.closed_form(values.double().cpu().numpy(), query.double().cpu().numpy())
    exact = torch.from_numpy(exact).cuda()
    # FP32 arithmetic leaves a few 1e-6 of absolute error in the logits' softmax; beyond
    # that the pair is good to FP32 rounding (S fused multiply-adds), the BF16 output alone
    # only to 2^-9.
    one = (out.double() - exact).abs()
    two = (joined.double() - exact).abs()
    assert bool((two <= 2.0**-21 * exact.abs() + 4e-6).all()), two.max().item()
    assert two.max().item() < one.max().item() / 64, (one.max().item(), two.max().item())


STREAM_SHAPES = [
    (49, 2000, 2048, 2048), (49, 1400, 4096, 4096), (17, 1400, 4096, 4096),
    (97, 1000, 4096, 64), (129, 500, 8192, 8192), (129, 500, 8192, 1024),
    (33, 2500, 1536, 128), (49, 2500, 1024, 1024), (5, 3000, 1024, 1024), (7, 700, 256, 256),
    (6, 2000, 3072, 3064),
]


@pytest.mark.parametrize("shape", STREAM_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_one_pass_backward_matches_the_oracle_and_the_two_pass_kernels(shape):
    """The streaming backward (several positions per warp group, so the ring wraps and the
    logits buffers rotate) against the oracle and against the staged kernels."""
    from attnres import _native
    torch.manual_seed(20261125)
    s, n, d, r = shape
    values = torch.randn(s, n, d, device="cuda", dtype=BF16)
    query = torch.randn(r, device="cuda", dtype=BF16) * (0.02 if r == d else 0.25)
    upstream = torch.randn(n, d, device="cuda", dtype=BF16)
    scale = 1.0 if r == d else r ** -0.5
    out, _, dv, dq = _abi_forward_backward(values, query, upstream, scale=scale, save=True,
                                           flags=_native.FLAG_PREFER_STREAM)
    out2, _, dv2, dq2 = _abi_forward_backward(values, query, upstream, scale=scale, save=False,
                                              flags=0)
    assert torch.equal(out, out2)
    e_out, e_dv, e_dq = ao.oracle_with_grads(values, query, upstream, scale=scale)
    _check_triplet((out, dv, dq.to(BF16)), (e_out, e_dv, e_dq))
    # the two kernels round the same FP32 quantities: they differ by single BF16 ulps
    assert ((dv.float() - dv2.float()).abs() <= 2.0**-6 * dv2.float().abs() + 1e-3).all()
    torch.testing.assert_close(dq, dq2, rtol=2e-3, atol=2e-3 * dq2.abs().max().item())
    assert _native.error_flag() == 0


def test_no_kernel_gave_up_waiting():
    """The bounded barrier waits of the TMA-staged kernels never expired in this process."""
    from attnres import _native
    torch.cuda.synchronize()
    assert _native.error_flag() == 0


def test_a_wait_that_runs_out_raises_the_flag_and_the_kernel_returns():
    """The give-up path of the kernels' bounded barrier wait, run by the library's self-test:
    one CTA announces 32 bytes, copies 16 and waits with a limit of one millisecond.  The
    kernel must return (no hang), the sticky device flag must read 1, and clearing it works.
    Nothing faults: the wait simply runs out."""
    from attnres import _native
    torch.cuda.synchronize()
    assert _native.error_flag() == 0
    scratch = torch.zeros(64, device="cuda", dtype=torch.uint8)
    _native.selftest_wait_limit(scratch.data_ptr(), 1_000_000,
                                torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _native.error_flag(clear=True) == 1
    assert _native.error_flag() == 0
    # the context is intact: an ordinary call still works and raises nothing
    from attnres import attnres
    values = torch.randn(3, 16, 256, device="cuda", dtype=BF16)
    query = torch.randn(256, device="cuda", dtype=BF16) * 0.1
    out = attnres(values, query)
    torch.testing.assert_close(out, ao.oracle(values, query), **TOL)
    assert _native.error_flag() == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from attnres import _native
    monkeypatch.setattr(_native, "_library", None)
    monkeypatch.setattr(_native, "LIBRARY_PATH", tmp_path / "absent.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _native.load()


def test_in_place_update_of_a_saved_output_is_refused_not_miscomputed():
    """Where the one-pass backward keeps the output, an in-place update of it between forward
    and backward must raise (autograd's version check), never give gradients of stale data."""
    from attnres import _native, attnres
    torch.manual_seed(2)
    shape = (9, 64, 2048, 2048)
    assert _native.wants_output_residual(shape[0], shape[2], shape[3])
    values = torch.randn(shape[0], shape[1], shape[2], device="cuda", dtype=BF16, requires_grad=True)
    query = (torch.randn(shape[3], device="cuda", dtype=BF16) * 0.02).requires_grad_()
    out = attnres(values, query)
    out.add_(1.0)
    with pytest.raises(RuntimeError, match="inplace"):
        out.sum().backward()
    # the out-of-place form is fine
    out = attnres(values, query)
    (out + 1.0).sum().backward()
    assert values.grad is not None and torch.isfinite(values.grad).all()
