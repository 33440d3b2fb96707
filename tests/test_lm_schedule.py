"""The benchmark language model's source schedules and its data-parallel step, on CPU with the
oracle as the read (the model is scaffolding for the benchmark's model workloads; the schedule
counts are the reference's, tests/test_training.py:109-131 and benchmarks/run.py:687-739)."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from baseline import lm  # noqa: E402
from oracle import attnres_oracle as ao  # noqa: E402


def _oracle_read(values, query):
    return ao.oracle(values, query)


def test_full_schedule_reads_every_earlier_output():
    config = lm.LMConfig(layers=24, width=1024, heads=16, ffn=4096, mode="full")
    counts = lm.read_source_counts(config)
    assert counts == tuple(range(2, 50)) and len(counts) == 48 and sum(counts) == 1224
    # the 24-layer Full-schedule step (S = 2..49, D = 1024): 126.4 GB of AttnRes traffic at 16 384 rows
    assert abs(lm.attnres_algorithmic_bytes(config, 16384) / 1e9 - 126.4) < 0.1


def test_block_schedule_counts():
    tiny = lm.LMConfig(layers=2, width=16, heads=4, ffn=32, mode="block", block_layers=1)
    assert lm.read_source_counts(tiny) == (2, 2, 3, 3)
    # 24 layers in blocks of 4: 48 reads, eight each with 2..7 sources
    config = lm.LMConfig(layers=24, width=4096, heads=32, ffn=16384, rank=1024, mode="block",
                         block_layers=4)
    counts = lm.read_source_counts(config)
    assert len(counts) == 48 and sum(counts) == 216 and max(counts) == 7
    assert [counts.count(s) for s in range(2, 8)] == [8] * 6


@pytest.mark.parametrize("layout", ["list", "packed"])
@pytest.mark.parametrize("mode", ["full", "block"])
def test_model_calls_the_operator_with_the_scheduled_sources(mode, layout):
    torch.manual_seed(3)
    config = lm.LMConfig(layers=2, width=16, heads=4, ffn=32, vocab=31, sequence=8, rank=4,
                         mode=mode, block_layers=1, layout=layout)
    seen = []

    def operator(values, query):
        seen.append(len(values))
        assert isinstance(values, tuple) == (layout == "list")
        return ao.oracle(values, query)

    model = lm.CausalLM(config, operator)
    tokens = torch.randint(31, (2, 8))
    logits = model(tokens)
    assert logits.shape == (2, 8, 31)
    assert tuple(seen) == lm.read_source_counts(config)
    logits.float().sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


def test_fused_norm_hook_replaces_read_plus_layernorm():
    torch.manual_seed(4)
    config = lm.LMConfig(layers=2, width=16, heads=4, ffn=32, vocab=31, sequence=8, mode="block",
                         block_layers=1)

    def normed(values, query, weight, bias, eps):
        out = ao.oracle(values, query)
        return torch.nn.functional.layer_norm(out.float(), (16,), weight, bias, eps)

    plain = lm.CausalLM(config, _oracle_read)
    fused = lm.CausalLM(config, _oracle_read, normed_operator=normed)
    fused.load_state_dict(plain.state_dict())
    tokens = torch.randint(31, (2, 8))
    torch.testing.assert_close(fused(tokens), plain(tokens))


def _free_port() -> int:
    import socket
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _ddp_worker(rank, world, port, state, tokens, targets, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        config = lm.LMConfig(layers=2, width=16, heads=4, ffn=32, vocab=31, sequence=8, rank=8,
                             mode="block", block_layers=1)
        model = lm.CausalLM(config, _oracle_read)
        model.load_state_dict(state)
        wrapped = torch.nn.parallel.DistributedDataParallel(model)
        optimizer = torch.optim.AdamW(model.parameters(), lr=1e-2)
        share = slice(rank * 2, rank * 2 + 2)
        lm.training_step(wrapped, optimizer, tokens[share], targets[share])
        results[rank] = {k: v.detach().clone() for k, v in model.state_dict().items()}
    finally:
        dist.destroy_process_group()


def test_data_parallel_step_equals_the_accumulated_single_process_step():
    """Two gloo ranks, each with its own half of the batch, one optimiser step under
    DistributedDataParallel (weight gradients and the [R] query gradients ride the same
    bucketed all-reduce) against one process accumulating the same two halves."""
    torch.manual_seed(1)
    config = lm.LMConfig(layers=2, width=16, heads=4, ffn=32, vocab=31, sequence=8, rank=8,
                         mode="block", block_layers=1)
    model = lm.CausalLM(config, _oracle_read)
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    tokens, targets = torch.randint(31, (4, 8)), torch.randint(31, (4, 8))
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-2)
    lm.training_step(model, optimizer, tokens, targets, accumulation=2)
    expected = model.state_dict()

    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_ddp_worker, args=(2, _free_port(), state, tokens, targets, results), nprocs=2,
             join=True)
    for rank in range(2):
        for name, value in expected.items():
            torch.testing.assert_close(results[rank][name], value, rtol=2e-3, atol=2e-5, msg=name)
