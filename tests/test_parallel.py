"""Shard arithmetic and the optional output all-gather, with two gloo ranks on the CPU."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sparta_b200 import parallel


def test_shard_bounds_cover_everything_once():
    for total, world, mult in [(4096, 8, 128), (2048, 4, 1), (64, 3, 1), (640, 4, 32), (7, 7, 1)]:
        spans = [parallel.shard_bounds(total, world, r, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c and a < b
        assert all((b - a) % mult == 0 for a, b in spans)
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= mult


def test_shard_bounds_errors():
    with pytest.raises(ValueError):
        parallel.shard_bounds(100, 4, 0, 32)      # not a multiple of the row tile
    with pytest.raises(ValueError):
        parallel.shard_bounds(64, 4, 0, 32)       # fewer groups than ranks
    with pytest.raises(ValueError):
        parallel.shard_bounds(64, 2, 2, 1)        # rank out of range


def _worker(rank, world, port, uneven):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        heads = 5 if uneven else 6
        q = torch.arange(heads * 4 * 3, dtype=torch.float32).reshape(heads, 4, 3)
        k = q + 1000
        ql, kl = parallel.shard_heads(q, k, world_size=world, rank=rank)
        lo, hi = parallel.shard_bounds(heads, world, rank)
        assert torch.equal(ql, q[lo:hi]) and torch.equal(kl, k[lo:hi])
        out = parallel.all_gather_outputs(ql * 2)       # stands in for the per-rank operator output
        assert torch.equal(out, q * 2)
        x = torch.arange(256 * 8, dtype=torch.float32).reshape(256, 8)
        xl = parallel.shard_rows(x, world, rank, block_rows=32)
        assert xl.shape[0] % 32 == 0
        assert torch.equal(parallel.all_gather_outputs(xl + 1), x + 1)
        m = (x > 100).to(torch.uint8)
        assert torch.equal(parallel.shard_row_mask(m, world, rank, 32), m[rank * 128:(rank + 1) * 128])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('uneven', [False, True])
def test_two_rank_shard_and_gather(uneven):
    port = 29500 + (os.getpid() % 2000) + (1 if uneven else 0)
    mp.spawn(_worker, args=(2, port, uneven), nprocs=2, join=True)
