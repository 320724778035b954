"""Two real GPUs over NCCL: the sharded, overlapped step leaves every rank with the parameters of
the unsharded step, bit for bit.  Skipped with fewer than two GPUs."""
import os
import random

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, name, steps, flat, exchange):
    import torch.distributed as dist
    from ista_daslab_optimizers_b200 import MicroAdam
    from ista_daslab_optimizers_b200.sharding import ShardedMicroAdam, flatten_parameters
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        case = cases.CASES[name]
        kw = dict(m=case.m, lr=case.lr, quant_block_size=case.qbs, k_init=case.k_init, alpha=case.alpha, betas=case.betas,
                  weight_decay=case.weight_decay, eps=case.eps, d_block_size=case.d_block_size)
        ref_params = [torch.nn.Parameter(p.cuda()) for p in case.params()]
        ref = MicroAdam(ref_params, **kw)
        params = [torch.nn.Parameter(p.cuda()) for p in case.params()]
        if flat:
            flatten_parameters(params)
        opt = ShardedMicroAdam(params, overlap_chunks=3, exchange=exchange, **kw)
        for t in range(steps):
            grads = case.grads(t)
            for p, q, g in zip(ref_params, params, grads):
                p.grad = g.cuda()
                q.grad = g.cuda()
            ref.step()
            opt.step()
            torch.cuda.synchronize()
            for i, (p, q) in enumerate(zip(ref_params, params)):
                assert torch.equal(p.detach().view(torch.int16 if p.dtype == torch.bfloat16 else torch.int32),
                                   q.detach().view(torch.int16 if q.dtype == torch.bfloat16 else torch.int32)), (rank, t, i)
        assert opt.last_gather_bytes > 0
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
@pytest.mark.parametrize('name,flat,exchange', [('bf16_wd', True, 'params'), ('mixed_fp32_alpha', False, 'params'), ('bf16_wd', False, 'rows')])
def test_two_gpus_match_one(name, flat, exchange):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, 29600 + random.randrange(2000), name, 3, flat, exchange), nprocs=2, join=True)


def _reduce_worker(rank, world, port, flat):
    """Gradient side of the shard plan on NCCL: every planned range summed into its owner."""
    import torch.distributed as dist
    from ista_daslab_optimizers_b200.sharding import plan_shards, reduce_to_owners, flatten_parameters
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        dbs = 29056
        # flat: sizes that are multiples of 64 elements leave no padding between the views, so a rank's ranges merge into one
        numels = [5120, 3 * dbs + 128, 64, 2 * dbs] if flat else [5000, 3 * dbs + 100, 64, 2 * dbs]
        plan = plan_shards(numels, dbs, 64, world)
        # rank r contributes (r + 1) * (position + 1) + tensor index
        grads = [(rank + 1) * (torch.arange(n, dtype=torch.float32, device='cuda') + 1) + i for i, n in enumerate(numels)]
        if flat:
            holders = [torch.nn.Parameter(g, requires_grad=False) for g in grads]
            flatten_parameters(holders)
            grads = [h.data for h in holders]
        owned = reduce_to_owners(plan, grads, rank, world, None, average=True)
        torch.cuda.synchronize()
        assert owned == 4 * sum(pc.hi - pc.lo for pc in plan if pc.rank == rank)
        mean_factor = sum(r + 1 for r in range(world)) / world
        for pc in plan:
            if pc.rank == rank:                             # only the owner's copy of a range is defined afterwards
                want = mean_factor * (torch.arange(pc.lo, pc.hi, dtype=torch.float32, device='cuda') + 1) + pc.index
                torch.testing.assert_close(grads[pc.index][pc.lo:pc.hi], want, rtol=1e-6, atol=1e-6)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
@pytest.mark.parametrize('flat', [True, False], ids=['one_reduce_scatter', 'reduce_per_view'])
def test_two_gpus_reduce_gradients_to_owners(flat):
    import torch.multiprocessing as mp
    mp.spawn(_reduce_worker, args=(2, 29600 + random.randrange(2000), flat), nprocs=2, join=True)
