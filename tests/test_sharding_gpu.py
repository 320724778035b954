"""A sharded step equals the unsharded step bit for bit (each rank's shard run in turn on one GPU)."""
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def bits(t):
    return t.detach().cpu().contiguous().view(torch.uint8) if t.dtype != torch.uint8 else t.detach().cpu()


@pytest.mark.parametrize('world', [2, 3])
@pytest.mark.parametrize('name', ['bf16_wd', 'mixed_fp32_alpha'])
def test_sharded_equals_unsharded(name, world):
    from ista_daslab_optimizers_b200.sharding import ShardedMicroAdam
    case = cases.CASES[name]
    full = cases.CudaAdapter(case, case.params())
    kw = dict(m=case.m, lr=case.lr, quant_block_size=case.qbs, k_init=case.k_init, alpha=case.alpha, betas=case.betas,
              weight_decay=case.weight_decay, eps=case.eps, d_block_size=case.d_block_size)
    ranks = []
    for r in range(world):
        params = [torch.nn.Parameter(p.cuda()) for p in case.params()]
        ranks.append((params, ShardedMicroAdam(params, rank=r, world_size=world, gather=False, **kw)))
    plan = ranks[0][1].plan
    assert {pc.rank for pc in plan} == set(range(world))
    qbs, m = case.qbs, case.m
    for t in range(4):
        grads = case.grads(t)
        full.step(grads)
        for params, opt in ranks:
            for p, g in zip(params, grads):
                p.grad = g.cuda()
            opt.step()
        for pc in plan:
            params, opt = ranks[pc.rank]
            su, sr = full.state(pc.index), opt.state[params[pc.index]]
            dbs, k_many = su['d_block_size'], su['k_block_size_many']
            assert sr['d'] == pc.hi - pc.lo
            row = (su['index'] - 1) % m
            c0 = (pc.lo // dbs) * k_many
            assert torch.equal(su['I'][row, c0:c0 + sr['k']], sr['I'][row])
            assert torch.equal(bits(su['V'][row, c0:c0 + sr['k']]), bits(sr['V'][row]))
            assert torch.equal(su['error'][pc.lo // 2:(pc.hi + 1) // 2], sr['error'])
            used = (sr['d'] + qbs - 1) // qbs
            q0 = pc.lo // qbs
            assert torch.equal(bits(su['min_vals'][q0:q0 + used]), bits(sr['min_vals'][:used]))
            assert torch.equal(bits(su['max_vals'][q0:q0 + used]), bits(sr['max_vals'][:used]))
            assert torch.equal(bits(full.param(pc.index).view(-1)[pc.lo:pc.hi]), bits(params[pc.index].data.view(-1)[pc.lo:pc.hi]))


@pytest.mark.parametrize('world', [1, 2, 3])
@pytest.mark.parametrize('name', ['bf16_wd', 'c1_fp32_1m'])
def test_row_exchange_equals_unsharded(name, world):
    """exchange='rows': kernel A sharded, window rows exchanged (copied by hand between the emulated
    ranks here), kernel B on every rank over all parameters: every rank ends with the unsharded result."""
    from ista_daslab_optimizers_b200.sharding import ShardedMicroAdam
    case = cases.CASES[name]
    full = cases.CudaAdapter(case, case.params())
    kw = dict(m=case.m, lr=case.lr, quant_block_size=case.qbs, k_init=case.k_init, alpha=case.alpha, betas=case.betas,
              weight_decay=case.weight_decay, eps=case.eps, d_block_size=case.d_block_size)
    ranks = []
    for r in range(world):
        params = [torch.nn.Parameter(p.cuda()) for p in case.params()]
        ranks.append((params, ShardedMicroAdam(params, rank=r, world_size=world, gather=False, exchange='rows', **kw)))
    for t in range(case.m + 2):
        grads = case.grads(t)
        full.step(grads)
        for params, opt in ranks:
            for p, g in zip(params, grads):
                p.grad = g.cuda()
            opt.steps += 1
            opt.rows_prepare()
            opt.rows_phase_a()
        for r_src, (_, src) in enumerate(ranks):
            for r_dst, (_, dst) in enumerate(ranks):
                if r_dst != r_src:
                    for a, b in zip(src.row_views()[r_src], dst.row_views()[r_src]):
                        b.copy_(a)
        for params, opt in ranks:
            opt.rows_phase_b()
            for i, p in enumerate(params):
                su, sr = full.state(i), opt.state[p]
                row = (su['index'] - 1) % case.m
                assert torch.equal(su['I'][row], sr['I'][row]), (t, i)
                assert torch.equal(bits(su['V'][row]), bits(sr['V'][row])), (t, i)
                assert torch.equal(bits(full.param(i)), bits(p.data)), (t, i)
        for pc in ranks[0][1].plan:
            params, opt = ranks[pc.rank]
            su, sr = full.state(pc.index), opt.state[params[pc.index]]
            assert torch.equal(su['error'][pc.lo // 2:(pc.hi + 1) // 2], sr['error'])
