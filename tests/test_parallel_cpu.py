"""Position sharding on CPU ranks (gloo, world size 2): the row partition and the
FP32 query-gradient all-reduce, with the oracle's closed form standing in for the
kernels.  The reference has no distributed code; these tests cover the new N > 1 path."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from attnres.parallel import all_reduce_query_grad, shard_rows
from oracle import attnres_oracle as ao


@pytest.mark.parametrize("rows,world", [(16384, 8), (10, 3), (7, 8), (0, 2), (1, 1), (131072, 4)])
def test_shard_rows_is_a_partition(rows, world):
    ranges = [shard_rows(rows, world, rank) for rank in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == rows
    for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
        assert a1 == b0 and a0 <= a1
    sizes = [stop - start for start, stop in ranges]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def test_shard_rows_rejects_bad_ranks():
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)
    with pytest.raises(ValueError):
        shard_rows(8, 0, 0)
    with pytest.raises(ValueError):
        shard_rows(-1, 2, 0)


def test_query_grad_reduction_requires_fp32():
    with pytest.raises(TypeError):
        all_reduce_query_grad(torch.zeros(4, dtype=torch.bfloat16))
    # without a process group the call is the BF16 rounding alone
    out = all_reduce_query_grad(torch.tensor([1.0, 2.00390625]))
    assert out.dtype == torch.bfloat16 and out.tolist() == [1.0, 2.0]


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _inputs():
    generator = torch.Generator().manual_seed(20260827)
    values = torch.randn(5, 37, 64, generator=generator).to(torch.bfloat16)
    query = (torch.randn(16, generator=generator) * 0.25).to(torch.bfloat16)
    upstream = torch.randn(37, 64, generator=generator).to(torch.bfloat16)
    return values, query, upstream


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        values, query, upstream = _inputs()
        start, stop = shard_rows(values.shape[1], world, rank)
        out, dv, dq = ao.closed_form(values[:, start:stop].float().numpy(), query.float().numpy(),
                                     upstream[start:stop].float().numpy(), scale=0.25)
        reduced = all_reduce_query_grad(torch.from_numpy(dq).float())
        results[rank] = (start, stop, out, dv, reduced)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_reproduces_the_unsharded_read():
    world, port = 2, _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    values, query, upstream = _inputs()
    out, dv, dq = ao.closed_form(values.float().numpy(), query.float().numpy(),
                                 upstream.float().numpy(), scale=0.25)
    for rank in range(world):
        start, stop, out_r, dv_r, dq_r = results[rank]
        np.testing.assert_allclose(out_r, out[start:stop], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(dv_r, dv[:, start:stop], rtol=1e-12, atol=1e-12)
        # every rank holds the same reduced gradient, equal to the unsharded one after rounding
        assert dq_r.dtype == torch.bfloat16
        assert torch.equal(dq_r, results[0][4])
        torch.testing.assert_close(dq_r.float(), torch.from_numpy(dq).float(), rtol=2**-7, atol=1e-3)
