"""The read with the consumer's LayerNorm in its epilogue (`attnres.fused.attnres_layer_norm`)
against the composition it replaces: LayerNorm applied to the read's BF16 result
(benchmarks/model.py:156, 170 of the reference), forward and backward, for every kernel family."""
import pytest
import torch
import torch.nn.functional as F

from oracle import attnres_oracle as ao

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
TOL = dict(rtol=0.05, atol=0.05)


@pytest.fixture(params=["auto", "generic", "stream"])
def family(request):
    from attnres import _native, _ops
    flags = {"auto": 0, "generic": _native.FLAG_FORCE_GENERIC,
             "stream": _native.FLAG_PREFER_STREAM}[request.param]
    previous = _ops.set_kernel_flags(flags)
    yield request.param
    _ops.set_kernel_flags(previous)


SHAPES = [(5, 37, 1024, 1024), (9, 300, 2048, 2048), (7, 129, 4096, 1024), (3, 11, 200, 72),
          (17, 65, 8192, 8192), (2, 500, 256, 256), (9, 33, 3000, 127)]


@pytest.mark.parametrize("as_list", [False, True], ids=["packed", "list"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_fused_layer_norm_matches_read_then_layer_norm(shape, as_list, family):
    from attnres import attnres
    from attnres.fused import attnres_layer_norm
    torch.manual_seed(20260827)
    s, n, d, r = shape
    values = torch.randn(s, n, d, device="cuda", dtype=BF16, requires_grad=True)
    query = (torch.randn(r, device="cuda", dtype=BF16) * 0.25).requires_grad_()
    weight = (1.0 + 0.1 * torch.randn(d, device="cuda")).requires_grad_()
    bias = (0.1 * torch.randn(d, device="cuda")).requires_grad_()
    upstream = torch.randn(n, d, device="cuda", dtype=BF16)
    side = torch.randn(n, d, device="cuda", dtype=BF16)     # a second consumer of the plain read
    leaves = (values, query, weight, bias)
    arg = tuple(values.unbind(0)) if as_list else values
    scale = 1.0 if r == d else r ** -0.5

    normed, read = attnres_layer_norm(arg, query, weight, bias, 1e-5, scale=scale, return_read=True)
    assert normed.dtype == BF16 and read.dtype == BF16
    got = torch.autograd.grad((normed, read), leaves, (upstream, side))

    # the composition it replaces, with this library's own read ...
    plain = attnres(arg, query, scale=scale)
    assert torch.equal(read, plain)
    composed = F.layer_norm(plain.float(), (d,), weight, bias, 1e-5)
    want = torch.autograd.grad((composed, plain), leaves, (upstream.float(), side))
    # the forward differs from it by the rounding of the result to BF16 only
    torch.testing.assert_close(normed.float(), composed, rtol=2**-7, atol=2**-7)
    for name, a, e in zip(("dvalues", "dquery", "dweight", "dbias"), got, want):
        assert torch.isfinite(a.float()).all(), name
        scale_of = float(e.float().abs().max()) + 1e-6
        torch.testing.assert_close(a.float(), e.float(), rtol=0.05, atol=0.05 * max(1.0, scale_of),
                                   msg=name)
        metrics = ao.error_metrics(a, e)
        assert metrics["relative_l2"] < 2e-2, (name, metrics)
    # ... and with the oracle as the read
    reference = ao.oracle(values, query, scale=scale)
    expected = F.layer_norm(reference.float(), (d,), weight, bias, 1e-5)
    torch.testing.assert_close(normed.float(), expected, **TOL)


def test_fused_layer_norm_without_affine_parameters_and_under_compile():
    from attnres.fused import attnres_layer_norm
    torch.manual_seed(3)
    values = [torch.randn(4, 64, 1024, device="cuda", dtype=BF16, requires_grad=True)
              for _ in range(6)]
    query = (torch.randn(1024, device="cuda", dtype=BF16) * 0.1).requires_grad_()
    eager = attnres_layer_norm(values, query)
    torch.testing.assert_close(eager.float().mean(-1), torch.zeros(4, 64, device="cuda"),
                               atol=2e-2, rtol=0)
    torch.testing.assert_close(eager.float().std(-1, unbiased=False),
                               torch.ones(4, 64, device="cuda"), atol=2e-2, rtol=0)

    @torch.compile(fullgraph=True, dynamic=False)
    def compiled(sources, q):
        return attnres_layer_norm(sources, q).float().square().mean()

    loss = compiled(values, query)
    grads = torch.autograd.grad(loss, (*values, query))
    expected = torch.autograd.grad(attnres_layer_norm(values, query).float().square().mean(),
                                   (*values, query))
    for a, e in zip(grads, expected):
        torch.testing.assert_close(a.float(), e.float(), rtol=0.05, atol=1e-4)


def test_fused_layer_norm_c_abi_writes_only_its_outputs():
    """Raw call with guard bands around the two extra outputs."""
    from attnres import _native
    torch.manual_seed(5)
    s, n, d, r = 5, 37, 1024, 512
    values = torch.randn(s, n, d, device="cuda", dtype=BF16)
    query = torch.randn(r, device="cuda", dtype=BF16) * 0.25
    weight = torch.randn(d, device="cuda")
    bias = torch.randn(d, device="cuda")
    pad = 256

    def guarded(numel, dtype):
        whole = torch.full((numel + 2 * pad,), -7, device="cuda", dtype=dtype)
        return whole, whole[pad:pad + numel]

    out_w, out = guarded(n * d, BF16)
    normed_w, normed = guarded(n * d, BF16)
    nstat_w, nstats = guarded(2 * n, torch.float32)
    logits = torch.empty(s, n, device="cuda", dtype=torch.float32)
    stats = torch.empty(2, n, device="cuda", dtype=torch.float32)
    step = n * d * 2
    for flags in (0, _native.FLAG_FORCE_GENERIC):
        _native.forward_layer_norm([values.data_ptr() + i * step for i in range(s)], [d] * s,
                                   [1] * s, s, n, d, r, query.data_ptr(), 1, 2**-23, 1.0,
                                   out.data_ptr(), d, logits.data_ptr(), stats.data_ptr(),
                                   weight.data_ptr(), bias.data_ptr(), 1e-5, normed.data_ptr(),
                                   nstats.data_ptr(), flags, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        for whole in (out_w, normed_w, nstat_w):
            assert bool((whole[:pad] == -7).all()) and bool((whole[-pad:] == -7).all())
        x = out.view(n, d).float()
        torch.testing.assert_close(nstats[:n], x.mean(-1), rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(nstats[n:], torch.rsqrt(x.var(-1, unbiased=False) + 1e-5),
                                   rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(normed.view(n, d).float(),
                                   F.layer_norm(x, (d,), weight, bias, 1e-5), rtol=2**-7, atol=2**-7)


@pytest.mark.parametrize("rows,width", [(37, 1024), (300, 2048), (129, 4096), (65, 8192), (500, 256),
                                        (33, 3000),
                                        # more rows than one pass of the grid: every CTA goes
                                        # round its shared-memory ring more than once
                                        (9001, 1024), (3001, 2048), (2001, 4096), (701, 8192)])
def test_layer_norm_backward_kernel_matches_the_framework(rows, width):
    """The library's LayerNorm-backward kernel (the backward of the fused epilogue) against
    autograd through F.layer_norm on the same BF16 read, for a contiguous and a strided
    upstream gradient."""
    from attnres.fused import layer_norm_backward
    torch.manual_seed(7)
    x = torch.randn(rows, width, device="cuda", dtype=BF16)
    weight = 1.0 + 0.1 * torch.randn(width, device="cuda")
    bias = 0.1 * torch.randn(width, device="cuda")
    mean = x.float().mean(-1)
    rstd = torch.rsqrt(x.float().var(-1, unbiased=False) + 1e-5)
    stats = torch.stack((mean, rstd)).contiguous()
    for grad in (torch.randn(rows, width, device="cuda", dtype=BF16),
                 torch.randn(rows, width + 8, device="cuda", dtype=BF16)[:, :width]):
        leaf = x.float().requires_grad_()
        w, b = weight.clone().requires_grad_(), bias.clone().requires_grad_()
        F.layer_norm(leaf, (width,), w, b, 1e-5).backward(grad.float())
        through, grad_weight, grad_bias = layer_norm_backward(grad, x, stats, weight)
        assert through.dtype == BF16 and grad_weight.dtype == torch.float32
        torch.testing.assert_close(through.float(), leaf.grad, rtol=2**-7, atol=2**-7)
        torch.testing.assert_close(grad_weight, w.grad, rtol=1e-3, atol=1e-3 * float(w.grad.abs().max()))
        torch.testing.assert_close(grad_bias, b.grad, rtol=1e-3, atol=1e-3 * float(b.grad.abs().max()))
