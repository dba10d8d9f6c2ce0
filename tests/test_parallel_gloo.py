"""Batch partition across ranks, exercised with two (and three) gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from trimkv_b200.parallel import gather_rows, generate_partitioned, partition_bounds


def test_partition_bounds_cover_every_request_once():
    for n in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = partition_bounds(n, world, r)
                assert 0 <= lo <= hi <= n
                seen += list(range(lo, hi))
            assert seen == list(range(n))
            sizes = [partition_bounds(n, world, r)[1] - partition_bounds(n, world, r)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        partition_bounds(4, 2, 2)


def _fake_generate(ids):
    # stands in for model.generate on this rank's requests: a pure function of each request's own tokens
    new = (ids.sum(dim=1, keepdim=True) * torch.arange(1, 4)) % 1000
    return torch.cat([ids, new], dim=1)


def _worker(rank, world, port, n_requests, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        ids = torch.randint(0, 100, (n_requests, 6))
        out = generate_partitioned(_fake_generate, ids)
        lo, hi = partition_bounds(n_requests, world, rank)
        block = gather_rows(torch.full((hi - lo, 2), rank, dtype=torch.int64), n_requests)
        q.put((rank, out, block))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,n_requests", [(2, 8), (2, 5), (3, 2)])
def test_partitioned_generation_equals_single_rank(world, n_requests):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_requests, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    torch.manual_seed(0)
    ids = torch.randint(0, 100, (n_requests, 6))
    want = _fake_generate(ids)
    for rank, out, block in results:
        assert torch.equal(out, want), rank          # same rows, same order, on every rank
        owners = torch.cat([torch.full((partition_bounds(n_requests, world, r)[1] - partition_bounds(n_requests, world, r)[0],),
                                       r) for r in range(world)])
        assert torch.equal(block[:, 0], owners)
