"""The oracle restatements against the reference's golden vectors and analytic cases."""
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attnres_oracle as ao
from oracle import c_port

GOLDEN = np.load(Path(__file__).parent / "golden" / "reference_oracle.npz")
NAMES = [str(name) for name in GOLDEN["names"]]


def _case(name):
    get = lambda key: GOLDEN[f"{name}.{key}"]
    eps, scale = (float(x) for x in get("eps_scale"))
    return (ao.from_bf16_bits(get("values")), ao.from_bf16_bits(get("query")),
            ao.from_bf16_bits(get("upstream")), ao.from_bf16_bits(get("out")),
            ao.from_bf16_bits(get("dv")), ao.from_bf16_bits(get("dq")), eps, scale)


def _ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in BF16 steps between two BF16 tensors (monotone integer mapping)."""
    def key(t):
        raw = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(raw < 0, -(raw & 0x7fff), raw)
    return (key(a) - key(b)).abs()


@pytest.mark.parametrize("name", NAMES)
def test_torch_restatement_matches_reference_oracle_bits(name):
    values, query, upstream, out, dv, dq, eps, scale = _case(name)
    got_out, got_dv, got_dq = ao.oracle_with_grads(values, query, upstream, eps=eps, scale=scale)
    for got, want in ((got_out, out), (got_dv, dv), (got_dq, dq)):
        distance = _ulp_distance(got, want)
        # Same operations in the same order: identical bits on one machine.  A
        # different CPU vector width may reorder a sum, so allow isolated 1-ulp flips.
        assert int(distance.max()) <= 1
        assert float((distance == 0).float().mean()) >= 0.999


@pytest.mark.parametrize("name", NAMES)
def test_list_form_equals_packed_form(name):
    values, query, _, out, _, _, eps, scale = _case(name)
    got = ao.oracle(tuple(values.unbind(0)), query, eps=eps, scale=scale)
    assert int(_ulp_distance(got, out).max()) <= 1


@pytest.mark.parametrize("name", NAMES)
def test_closed_form_gradient_matches_reference_autograd(name):
    values, query, upstream, out, dv, dq, eps, scale = _case(name)
    got_out, got_dv, got_dq = ao.closed_form(values.float().numpy(), query.float().numpy(),
                                             upstream.float().numpy(), eps=eps, scale=scale)
    for got, want in ((got_out, out), (got_dv, dv), (got_dq, dq)):
        got = torch.from_numpy(got).to(torch.bfloat16)
        torch.testing.assert_close(got.float(), want.float(), rtol=2**-7, atol=2e-3)
        assert float((_ulp_distance(got, want) <= 1).float().mean()) >= 0.9


@pytest.mark.parametrize("name", NAMES)
def test_c_port_matches_reference_oracle(name):
    values, query, upstream, out, dv, dq, eps, scale = _case(name)
    bits = ao.bf16_bits
    got_out = c_port.forward(bits(values), bits(query), eps, scale)
    got_dv, got_dq = c_port.backward(bits(values), bits(query), bits(upstream), eps, scale)
    for got, want in ((got_out, out), (got_dv, dv), (got_dq, dq)):
        got = ao.from_bf16_bits(got)
        torch.testing.assert_close(got.float(), want.float(), rtol=2**-7, atol=2e-3)
        assert float((_ulp_distance(got, want) <= 1).float().mean()) >= 0.9


def test_oracle_rejects_other_dtypes():
    # validation/oracle.py:10-11
    with pytest.raises(TypeError, match="BF16"):
        ao.oracle(torch.ones(2, 3, 16), torch.ones(16))


@pytest.mark.parametrize("as_list", [False, True])
def test_oracle_ignores_ambient_autocast(as_list):
    # tests/test_bf16_oracle.py:10-30 of the reference
    torch.manual_seed(19)
    values = torch.randn(5, 3, 17).to(torch.bfloat16).requires_grad_()
    query = torch.randn(7).to(torch.bfloat16).requires_grad_()
    upstream = torch.randn(3, 17).to(torch.bfloat16)
    results = []
    for enabled in (False, True):
        with torch.autocast(device_type="cpu", dtype=torch.bfloat16, enabled=enabled):
            out = ao.oracle(tuple(values.unbind()) if as_list else values, query, scale=0.7)
        results.append((out, *torch.autograd.grad(out, (values, query), upstream)))
    for a, b in zip(*results):
        assert a.dtype == torch.bfloat16
        assert torch.equal(a, b)


def _routing_fixture(kind):
    """Inputs in the numeric regimes of validation/routing_checks.py:11-37."""
    torch.manual_seed(20260906)
    sources, rows, width, rank = 4, 3, 32, 16
    values = torch.randn(sources, rows, width)
    values[..., :-rank] += torch.arange(sources)[:, None, None]
    query = torch.randn(rank) * 0.05
    upstream = torch.randn(rows, width)
    eps, scale = 2**-10, -0.75
    if kind == "zero_keys":
        values[..., -rank:] = 0
    elif kind == "zero_scale":
        scale = 0.0
    elif kind == "large_logits":
        values[..., -rank:] = 0
        values[..., -rank] = 1
        values[..., -rank + 1] = torch.tensor([-1.0, 1.0, -1.0, 1.0])[:, None]
        query.zero_()
        query[0], query[1] = 1.0, 2**-22
        scale = 2.0**20
    to = lambda t: t.to(torch.bfloat16)
    return to(values), to(query), to(upstream), eps, scale


def test_zero_keys_have_closed_form_tail_gradient_and_zero_query_gradient():
    # tests/test_routing_checks.py:10-24 of the reference
    values, query, upstream, eps, scale = _routing_fixture("zero_keys")
    _, dv, dq = ao.oracle_with_grads(values, query, upstream, eps=eps, scale=scale)
    v, g, q = values.float(), upstream.float(), query.float()
    dz = ((v - v.mean(0)) * g).sum(-1) / 4
    dk = scale * dz[..., None] * q / math.sqrt(eps)
    assert torch.count_nonzero(dk) == dk.numel()
    expected = (g[None, ..., -16:] / 4 + dk).to(torch.bfloat16)
    torch.testing.assert_close(dv[..., -16:], expected, rtol=0.05, atol=0.05)
    assert torch.equal(dq, torch.zeros_like(dq))
    # The closed form agrees.
    _, dv64, dq64 = ao.closed_form(v.numpy(), q.numpy(), g.numpy(), eps=eps, scale=scale)
    torch.testing.assert_close(torch.from_numpy(dv64[..., -16:]).float(), expected.float(),
                               rtol=0.05, atol=0.05)
    assert np.abs(dq64).max() == 0.0


def test_zero_scale_leaves_only_the_direct_gradient():
    # tests/test_routing_checks.py:39-47 of the reference
    values, query, upstream, eps, scale = _routing_fixture("zero_scale")
    _, dv, dq = ao.oracle_with_grads(values, query, upstream, eps=eps, scale=scale)
    assert torch.equal(dv, (upstream.expand_as(values) / 4))
    assert torch.equal(dq, torch.zeros_like(dq))


def test_large_logit_fixture_is_finite_and_not_uniform():
    # tests/test_routing_checks.py:27-36 of the reference
    values, query, _, eps, scale = _routing_fixture("large_logits")
    key = values[..., -16:].float()
    logits = (key * query.float()).sum(-1) * torch.rsqrt(key.square().mean(-1) + eps) * scale
    assert torch.isfinite(logits).all() and logits.min() > 1e6
    assert logits.unique().numel() == 2
    assert (logits.softmax(0) - 0.25).abs().max() > 0.01


@pytest.mark.parametrize("scale", [2**24, -(2**24)])
def test_max_and_normaliser_must_stay_separate(scale):
    # tests/test_softmax_stats.py:6-15 of the reference: a fused max+log(sum)
    # loses log(S) at |logit| ~ 2.7e8, which is why the kernels save (max, 1/sum).
    keys = torch.ones(4, 2, 16)
    logits = keys.sum(-1) * torch.rsqrt(keys.square().mean(-1) + 2**-23) * scale
    top = logits.max(0).values
    numerator = (logits - top).exp()
    denominator = numerator.sum(0)
    fused = (logits - (top + denominator.log())).exp()
    assert torch.equal(fused, torch.ones_like(fused))
    assert torch.equal(numerator / denominator, logits.softmax(0))


def test_equal_logits_give_exact_uniform_gradients():
    # validation/softmax_checks.py:26-30 of the reference
    values = torch.ones(4, 2, 256, dtype=torch.bfloat16)
    query = torch.ones(16, dtype=torch.bfloat16)
    upstream = torch.ones(2, 256, dtype=torch.bfloat16)
    out, dv, dq = ao.oracle_with_grads(values, query, upstream, scale=2.0**24)
    assert torch.equal(out, values[0])
    assert torch.equal(dv, upstream.expand_as(values) / 4)
    assert torch.equal(dq, torch.zeros_like(dq))


def test_error_metrics_follow_the_reference_definition():
    a = torch.tensor([1.0, 2.0, 4.0])
    b = torch.tensor([1.0, 2.5, 4.0])
    metrics = ao.error_metrics(a, b)
    assert metrics["max_abs"] == 0.5
    assert abs(metrics["relative_l2"] - 0.5 / math.sqrt(1 + 6.25 + 16)) < 1e-7
