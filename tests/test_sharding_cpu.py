"""Row sharding over ranks and the gather that completes it, on CPU ranks (gloo, world_size 2/3).

The product's multi-GPU path shards batch rows with the reference's chunk formula and completes
the output with an all-gather; here the same host logic runs with torch.distributed's gloo backend
and is checked against the oracle's restatement of the reference collective and its golden grid.
"""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kutacc_b200 import sharding
from oracle import cpu_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_chunk_formula():
    for x in (1, 7, 8, 1000, 1024):
        for world in (1, 2, 3, 4, 8):
            chunks = [sharding.chunk(x, world, r) for r in range(world)]
            assert sum(chunks) == x
            lo_hi = [sharding.row_range(x, world, r) for r in range(world)]
            assert lo_hi[0][0] == 0 and lo_hi[-1][1] == x
            for r in range(world - 1):
                assert lo_hi[r][1] == lo_hi[r + 1][0] or chunks[r + 1] == 0
    assert [sharding.chunk(1000, 8, r) for r in range(8)] == [125] * 8
    assert [sharding.chunk(7, 3, r) for r in range(3)] == [3, 3, 1]
    assert [sharding.chunk(5, 4, r) for r in range(4)] == [2, 2, 1, 0]       # an empty last rank is legal


def _worker(rank, world, port, m, n, ln, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = np.arange(m * n * ln, dtype=np.uint8).reshape(m, n, ln) if m * n * ln < 256 else \
            np.random.default_rng(0).integers(0, 255, (m, n, ln), dtype=np.uint8)
        lo, hi = sharding.row_range(m, world, rank)
        blk = sharding.block(m, world)
        mine = np.zeros((blk, n, ln), dtype=np.uint8)           # padded to the block size, as the library does
        mine[:hi - lo] = full[lo:hi]
        gathered = [torch.zeros((blk, n, ln), dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine))
        out = np.zeros((m, n, ln), dtype=np.uint8)
        for r in range(world):
            rlo, rhi = sharding.row_range(m, world, r)
            out[rlo:rhi] = gathered[r].numpy()[:rhi - rlo]
        ret[rank] = bool(np.array_equal(out, full))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,m,n,ln", [(2, 8, 5, 1), (2, 7, 6, 3), (3, 7, 4, 2)])
def test_sharded_rows_gather_back_on_gloo(world, m, n, ln):
    port = 29500 + (os.getpid() % 2000) + world * 7 + m
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, port, m, n, ln, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world))


def test_gloo_grid_equals_reference_golden():
    g = np.load(os.path.join(GOLD, "all_gather_grid.npz"))
    out = O.all_gather_bytes([g["shard0"], g["shard1"]], (8, 5, 1), data_size0=4)
    lo0, hi0 = sharding.row_range(8, 2, 0)
    lo1, hi1 = sharding.row_range(8, 2, 1)
    assert np.array_equal(out[lo0:hi0], g["shard0"]) and np.array_equal(out[lo1:hi1], g["shard1"])


def test_slab_plan_gives_every_row_to_exactly_one_rank():
    from kutacc_b200 import sharding
    for n, world, nslab in [(1024, 8, 2), (1024, 4, 4), (384, 2, 3), (128, 1, 2)]:
        seen = []
        for rank in range(world):
            own = sharding.owned_rows(n, world, rank, nslab)
            assert len(own) == nslab
            for (r0, cnt), (s0, srows, blk) in zip(own, sharding.slab_plan(n, world, nslab)):
                assert cnt == blk and s0 + rank * blk == r0 and r0 + cnt <= s0 + srows
                seen += list(range(r0, r0 + cnt))
        assert sorted(seen) == list(range(n))
    with pytest.raises(ValueError):
        sharding.slab_plan(1000, 8, 3)
