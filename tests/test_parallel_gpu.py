"""Position sharding on real GPUs: two ranks on two devices over NCCL (skipped on a one-GPU box),
and two ranks sharing ONE device over gloo, which runs everywhere.

Each rank runs the CUDA kernels on its own rows; the FP32 query gradients meet in one NCCL
all-reduce and are rounded to BF16 once.  The result must equal the unsharded read: outputs and
value gradients bit for bit (positions are independent), the query gradient within one BF16
rounding of the FP32 reassociation.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
needs_two_gpus = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _inputs(device):
    generator = torch.Generator(device="cpu").manual_seed(20260827)
    values = torch.randn(6, 1000, 1024, generator=generator).to(torch.bfloat16).to(device)
    query = (torch.randn(256, generator=generator) * 0.25).to(torch.bfloat16).to(device)
    upstream = torch.randn(1000, 1024, generator=generator).to(torch.bfloat16).to(device)
    return values, query, upstream


def _worker(rank, world, port, as_list, results, backend="nccl"):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    for entry in (root, root / "fast-attnres_b200"):
        if str(entry) not in sys.path:
            sys.path.insert(0, str(entry))
    from attnres.parallel import shard_rows, sharded_attnres
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    # NCCL wants one device per rank; over gloo (host-staged collectives, nothing in a kernel
    # waits for another rank) both ranks may share device 0.
    device_index = rank if backend == "nccl" else 0
    torch.cuda.set_device(device_index)
    if backend == "nccl":
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", device_index))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        values, query, upstream = _inputs(f"cuda:{device_index}")
        start, stop = shard_rows(values.shape[1], world, rank)
        mine = values[:, start:stop].contiguous().requires_grad_()
        q = query.clone().requires_grad_()
        arg = tuple(mine.unbind(0)) if as_list else mine
        out = sharded_attnres(arg, q, scale=0.0625)
        dv, dq = torch.autograd.grad(out, (mine, q), upstream[start:stop])
        torch.cuda.synchronize()
        # plain NumPy bit patterns: tensors do not travel through a Manager proxy
        bits = lambda t: t.detach().contiguous().view(torch.int16).cpu().numpy()
        results[rank] = (start, stop, bits(out), bits(dv), bits(dq))
    finally:
        dist.destroy_process_group()


def _check_against_unsharded(backend, as_list):
    from attnres import attnres
    world, port = 2, _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, as_list, results, backend), nprocs=world, join=True)
    values, query, upstream = _inputs("cuda:0")
    values.requires_grad_()
    query.requires_grad_()
    out = attnres(values, query, scale=0.0625)
    dv, dq = torch.autograd.grad(out, (values, query), upstream)
    back = lambda a: torch.from_numpy(a).view(torch.bfloat16)
    for rank in range(world):
        start, stop, out_r, dv_r, dq_r = results[rank]
        out_r, dv_r, dq_r = back(out_r), back(dv_r), back(dq_r)
        assert torch.equal(out_r, out[start:stop].cpu())
        assert torch.equal(dv_r, dv[:, start:stop].cpu())
        assert torch.equal(dq_r, back(results[0][4])), "ranks disagree on the reduced query gradient"
        torch.testing.assert_close(dq_r.float(), dq.cpu().float(), rtol=2**-7, atol=2**-7)


@needs_two_gpus
@pytest.mark.parametrize("as_list", [False, True], ids=["packed", "list"])
def test_two_gpu_sharding_equals_the_unsharded_read(as_list):
    _check_against_unsharded("nccl", as_list)


@pytest.mark.parametrize("as_list", [False, True], ids=["packed", "list"])
def test_two_ranks_on_one_gpu_equal_the_unsharded_read(as_list):
    """The same check with both ranks on device 0 and the FP32 query gradients summed over
    gloo: runs on a one-GPU box, so the sharded read's kernels and its collective are covered
    wherever the GPU tests run."""
    _check_against_unsharded("gloo", as_list)
