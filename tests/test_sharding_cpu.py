"""Shard planner and parameter exchange without a GPU (gloo, world size 2)."""
import os
import random

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ista_daslab_optimizers_b200.sharding import build_gather_views, exchange_pieces, plan_shards
from ista_daslab_optimizers_b200 import synthetic as S

DBS = 29056


def check_plan(numels, dbs, qbs, world):
    plan = plan_shards(numels, dbs, qbs, world)
    # every element exactly once, pieces in order
    covered = {i: 0 for i, n in enumerate(numels) if n}
    last_rank = 0
    for pc in plan:
        assert 0 <= pc.rank < world and pc.lo < pc.hi <= numels[pc.index]
        assert pc.lo == covered[pc.index], (pc, covered[pc.index])
        covered[pc.index] = pc.hi
        assert pc.rank >= last_rank                      # contiguous runs: ranks never go back
        last_rank = pc.rank
        d = numels[pc.index]
        splittable = d > dbs and dbs % qbs == 0
        if not splittable:
            assert (pc.lo, pc.hi) == (0, d)
        else:
            assert pc.lo % dbs == 0 and (pc.hi % dbs == 0 or pc.hi == d)
            assert pc.lo % qbs == 0
    assert all(covered[i] == n for i, n in enumerate(numels) if n)
    # at most one piece per (rank, tensor)
    assert len({(pc.rank, pc.index) for pc in plan}) == len(plan)
    return plan


def test_plan_llama_list_is_balanced():
    numels = [int(torch.Size(s).numel()) for s in S.llama3_8b_shapes()]
    total = sum(numels)
    for world in (1, 2, 4, 8):
        plan = check_plan(numels, DBS, 64, world)
        share = [0] * world
        for pc in plan:
            share[pc.rank] += pc.hi - pc.lo
        assert sum(share) == total
        # every cut is within one top-k block (or one unsplittable tensor) of the ideal
        assert max(abs(s - total / world) for s in share) <= max(DBS, 4096) + 1


def test_plan_random_lists():
    rng = random.Random(7)
    for _ in range(200):
        numels = [rng.choice([0, 1, 7, 64, 4096, DBS - 1, DBS, DBS + 1, 3 * DBS, 3 * DBS + 17, rng.randrange(1, 400000)])
                  for _ in range(rng.randrange(1, 12))]
        if sum(numels) == 0:
            continue
        for world in (1, 2, 3, 8):
            for qbs in (64, 100000):
                check_plan(numels, DBS, qbs, world)


def _worker(rank, world, port, numels, flat):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        plan = plan_shards(numels, DBS, 64, world)
        if flat:
            buf = torch.zeros(sum(numels))
            params, off = [], 0
            for n in numels:
                params.append(buf[off:off + n])
                off += n
        else:
            params = [torch.zeros(n) for n in numels]
        # every rank writes rank + 1 + position into the ranges it owns, as its "update"
        for pc in plan:
            if pc.rank == rank:
                params[pc.index][pc.lo:pc.hi] = torch.arange(pc.lo, pc.hi, dtype=torch.float32) + 1000.0 * (rank + 1)
        views = build_gather_views(plan, params, world)
        if flat:
            assert all(len(v) <= 1 for v in views)        # adjacent pieces were merged
        received = exchange_pieces(views, rank)
        mine = sum(pc.hi - pc.lo for pc in plan if pc.rank == rank)
        assert received == (sum(numels) - mine) * 4
        for pc in plan:
            want = torch.arange(pc.lo, pc.hi, dtype=torch.float32) + 1000.0 * (pc.rank + 1)
            assert torch.equal(params[pc.index][pc.lo:pc.hi], want), (rank, pc)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('flat', [False, True])
def test_exchange_gloo_world2(flat):
    numels = [5000, 3 * DBS + 100, 64, 2 * DBS]
    port = 29500 + random.randrange(2000)
    mp.spawn(_worker, args=(2, port, numels, flat), nprocs=2, join=True)


def _reduce_worker(rank, world, port, numels):
    from ista_daslab_optimizers_b200.sharding import reduce_to_owners
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        plan = plan_shards(numels, DBS, 64, world)
        # rank r contributes (r + 1) * (position + 1) + tensor index
        grads = [(rank + 1) * (torch.arange(n, dtype=torch.float32) + 1) + i for i, n in enumerate(numels)]
        owned = reduce_to_owners(plan, grads, rank, world, None, average=True)
        assert owned == 4 * sum(pc.hi - pc.lo for pc in plan if pc.rank == rank)
        mean_factor = sum(r + 1 for r in range(world)) / world
        for pc in plan:
            if pc.rank == rank:                             # only the owner's copy of a range is defined afterwards
                want = mean_factor * (torch.arange(pc.lo, pc.hi, dtype=torch.float32) + 1) + pc.index
                torch.testing.assert_close(grads[pc.index][pc.lo:pc.hi], want, rtol=1e-6, atol=1e-6)
    finally:
        dist.destroy_process_group()


def test_reduce_gradients_gloo_world2():
    numels = [5000, 3 * DBS + 100, 64, 2 * DBS]
    mp.spawn(_reduce_worker, args=(2, 29500 + random.randrange(2000), numels), nprocs=2, join=True)


def test_piece_geometry_matches_the_whole_tensor():
    """Kernel B of the 'rows' exchange describes every piece of the plan as a tensor of its own: a piece's own
    block geometry must select, block for block, what the whole tensor's geometry selects there."""
    from ista_daslab_optimizers_b200.sharding import block_geometry
    from ista_daslab_optimizers_b200 import synthetic as S
    shapes = S.llama3_8b_shapes()
    lists = [[5000, 3 * DBS + 100, 64, 2 * DBS, DBS, DBS + 1], [int(torch.Size(s).numel()) for s in shapes][:40]]
    for numels in lists:
        for world in (1, 2, 3, 8):
            plan = plan_shards(numels, DBS, 64, world)
            for idx, n in enumerate(numels):
                g = block_geometry(n, DBS, 0.01)
                pieces = [pc for pc in plan if pc.index == idx]
                assert sum(block_geometry(pc.hi - pc.lo, DBS, 0.01)['k'] for pc in pieces) == g['k']
                for pc in pieces:
                    sg = block_geometry(pc.hi - pc.lo, DBS, 0.01)
                    assert pc.lo % g['d_block_size'] == 0
                    first_col = (pc.lo // g['d_block_size']) * g['k_many']
                    end_col = g['k'] if pc.hi == n else (pc.hi // g['d_block_size']) * g['k_many']
                    assert first_col + sg['k'] == end_col, (n, pc)


def _gather_rows_worker(rank, world, port):
    from ista_daslab_optimizers_b200.sharding import gather_row_regions
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        row = torch.full((world, 192), -1, dtype=torch.int16)
        row[rank] = torch.arange(192, dtype=torch.int16) + 1000 * rank
        got = gather_row_regions(row, rank)
        assert got == (world - 1) * 192 * 2
        for r in range(world):
            assert torch.equal(row[r], torch.arange(192, dtype=torch.int16) + 1000 * r)
    finally:
        dist.destroy_process_group()


def test_gather_row_regions_gloo_world2():
    mp.spawn(_gather_rows_worker, args=(2, 29500 + random.randrange(2000)), nprocs=2, join=True)
