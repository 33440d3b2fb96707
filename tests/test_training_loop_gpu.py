"""A small Full-schedule network trained for a few steps through the public API: every layer
reads ALL earlier layer outputs with `attnres` (the schedule of the reference's benchmark model,
benchmarks/model.py:293-311), queries are `LearnedQuery` modules, the optimiser is AdamW.
The same network with the oracle in place of the operator is trained from the same weights
on the same data; the two loss curves must agree and fall."""
import copy

import pytest
import torch

from oracle import attnres_oracle as ao

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


class _FullScheduleNet(torch.nn.Module):
    def __init__(self, read, width, rank, layers):
        super().__init__()
        from attnres import LearnedQuery
        self.read, self.rank = read, rank
        self.queries = torch.nn.ModuleList(LearnedQuery(rank) for _ in range(layers))
        self.mix = torch.nn.ModuleList(torch.nn.Linear(width, width) for _ in range(layers))

    def forward(self, x, as_list):
        sources = [x]
        for query, mix in zip(self.queries, self.mix):
            values = tuple(sources) if as_list else torch.stack(sources)
            state = self.read(values, query(), scale=self.rank ** -0.5)
            sources.append(torch.tanh(mix(state)).to(BF16))
        return sources[-1]


@pytest.mark.parametrize("as_list", [False, True], ids=["packed", "list"])
def test_training_loop_follows_the_oracle_and_reduces_the_loss(as_list):
    from attnres import attnres
    torch.manual_seed(20260911)
    width, rank, layers, rows, steps = 512, 128, 6, 192, 12
    ours = _FullScheduleNet(attnres, width, rank, layers).cuda().to(BF16)
    for module in ours.queries:
        module.float()                      # FP32 master queries, BF16 on the wire
    twin = copy.deepcopy(ours)
    twin.read = lambda values, query, scale: ao.oracle(values, query, scale=scale)
    x = torch.randn(rows, width, device="cuda", dtype=BF16)
    target = torch.tanh(torch.randn(rows, width, device="cuda")).to(BF16)
    curves = []
    for net in (ours, twin):
        optimiser = torch.optim.AdamW(net.parameters(), lr=2e-3, weight_decay=0.0)
        losses = []
        for _ in range(steps):
            optimiser.zero_grad(set_to_none=True)
            loss = (net(x, as_list).float() - target.float()).square().mean()
            loss.backward()
            optimiser.step()
            losses.append(loss.item())
        curves.append(losses)
    mine, reference = curves
    assert mine[-1] < 0.7 * mine[0], mine
    for a, b in zip(mine, reference):
        assert abs(a - b) <= 0.05 * abs(b) + 1e-3, (mine, reference)
    for module in ours.queries:
        assert module.query.dtype == torch.float32 and module.query.grad.dtype == torch.float32
    # what a training loop should do at a step boundary: no kernel gave up a bounded wait
    from attnres import _native
    assert _native.error_flag() == 0
