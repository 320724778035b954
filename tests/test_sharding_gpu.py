"""A sharded step equals the unsharded step bit for bit (each rank's shard run in turn on one GPU)."""
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def bits(t):
    return t.detach().cpu().contiguous().view(torch.uint8) if t.dtype != torch.uint8 else t.detach().cpu()


@pytest.mark.parametrize('world', [2, 3])
@pytest.mark.parametrize('name', ['bf16_wd', 'mixed_fp32_alpha', 'qbs_100000_a0'])
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


def make_rows_ranks(case, world, **extra):
    from ista_daslab_optimizers_b200.sharding import ShardedMicroAdam
    kw = dict(m=case.m, lr=case.lr, quant_block_size=case.qbs, k_init=case.k_init, alpha=case.alpha, betas=case.betas,
              weight_decay=case.weight_decay, eps=case.eps, d_block_size=case.d_block_size)
    ranks = []
    for r in range(world):
        params = [torch.nn.Parameter(p.cuda()) for p in case.params()]
        ranks.append((params, ShardedMicroAdam(params, rank=r, world_size=world, gather=False, exchange='rows', **kw, **extra)))
    return ranks


def rows_step(ranks, grads, skip_grad=None):
    """One step of every emulated rank; the all-gather of the new row is done by hand (region r copied from rank r)."""
    for r, (params, opt) in enumerate(ranks):
        for i, (p, g) in enumerate(zip(params, grads)):
            p.grad = None if skip_grad and (r, i) in skip_grad else g.cuda()
        opt.steps += 1
        opt.rows_prepare()
        opt.rows_phase_a()
    for r_src, (_, src) in enumerate(ranks):
        for r_dst, (_, dst) in enumerate(ranks):
            if r_dst != r_src:
                dst.current_row()[r_src].copy_(src.current_row()[r_src])
    for _, opt in ranks:
        opt.rows_phase_b()


def assert_rows_ranks_equal_unsharded(case, full, ranks, t):
    for params, opt in ranks:
        for i, p in enumerate(params):
            assert torch.equal(bits(full.param(i)), bits(p.data)), (t, i)
    for pc in ranks[0][1].plan:
        params, opt = ranks[pc.rank]
        su, sr = full.state(pc.index), opt.state[params[pc.index]]
        row = (su['index'] - 1) % case.m
        c0 = (pc.lo // su['d_block_size']) * su['k_block_size_many']
        assert sr['index'] == su['index']
        assert torch.equal(su['I'][row, c0:c0 + sr['k']], sr['I'][row]), (t, pc)
        assert torch.equal(bits(su['V'][row, c0:c0 + sr['k']]), bits(sr['V'][row])), (t, pc)
        assert torch.equal(su['error'][pc.lo // 2:(pc.hi + 1) // 2], sr['error'])
    # the window is replicated: every rank holds the same buffer
    for _, opt in ranks[1:]:
        assert torch.equal(opt._window, ranks[0][1]._window)


@pytest.mark.parametrize('world', [1, 2, 3])
@pytest.mark.parametrize('name', ['bf16_wd', 'c1_fp32_1m', 'qbs_100000_a0_bf16'])
def test_row_exchange_equals_unsharded(name, world):
    """exchange='rows': kernel A sharded, window rows exchanged (copied by hand between the emulated
    ranks here), kernel B on every rank over all parameters: every rank ends with the unsharded result."""
    case = cases.CASES[name]
    full = cases.CudaAdapter(case, case.params())
    ranks = make_rows_ranks(case, world)
    for t in range(case.m + 2):
        grads = case.grads(t)
        full.step(grads)
        rows_step(ranks, grads)
        assert_rows_ranks_equal_unsharded(case, full, ranks, t)


def test_row_exchange_needs_gradients_of_owned_slices_only():
    """A rank may lack the gradient of a tensor it owns nothing of (kernel B still updates that tensor from the
    exchanged rows); lacking the gradient of an owned slice is an error, not a silent divergence."""
    case = cases.CASES['bf16_wd']
    full = cases.CudaAdapter(case, case.params())
    ranks = make_rows_ranks(case, 2)
    plan = ranks[0][1].plan
    owners = {i: {pc.rank for pc in plan if pc.index == i} for i in range(len(case.shapes))}
    not_owned = {(r, i) for r in range(2) for i in owners if r not in owners[i]}
    assert not_owned
    for t in range(3):
        grads = case.grads(t)
        full.step(grads)
        rows_step(ranks, grads, skip_grad=not_owned)
        assert_rows_ranks_equal_unsharded(case, full, ranks, t)
    r, i = next((r, i) for i in owners for r in owners[i])
    with pytest.raises(RuntimeError, match='no gradient'):
        rows_step(ranks, case.grads(3), skip_grad={(r, i)})


def test_row_exchange_checkpoint_resume():
    """'rows' mode: save after 3 steps, load into fresh optimizers (fresh parameters restored by the caller),
    3 more steps: bit-equal with the uninterrupted unsharded run."""
    case = cases.CASES['bf16_wd']
    full = cases.CudaAdapter(case, case.params())
    ranks = make_rows_ranks(case, 2)
    for t in range(3):
        grads = case.grads(t)
        full.step(grads)
        rows_step(ranks, grads)
    saved = [(opt.state_dict(), [p.detach().clone() for p in params]) for params, opt in ranks]
    assert all(sd['ring'] == 3 and sd['steps'] == 3 for sd, _ in saved)
    fresh = make_rows_ranks(case, 2)
    for (params, opt), (sd, values) in zip(fresh, saved):
        for p, v in zip(params, values):
            p.data.copy_(v)
        opt.load_state_dict(sd)
    with pytest.raises(ValueError):
        fresh[0][1].load_state_dict(saved[1][0])          # the other rank's checkpoint
    for t in range(3, 6):
        grads = case.grads(t)
        full.step(grads)
        rows_step(fresh, grads)
        assert_rows_ranks_equal_unsharded(case, full, fresh, t)


def test_row_exchange_logging_probes_add_up_to_the_unsharded_ones():
    """On a logging step every rank reports the probes of its own slices (gradient, error feedback) and rank 0 those of
    the update (which every rank computes alike); summed over the ranks, as the log does, they are the unsharded run's."""
    case = cases.CASES['bf16_wd']
    full = cases.CudaAdapter(case, case.params())
    full_log, rank_logs = [], [[], []]
    full.opt.log_fn, full.opt.log_interval = full_log.append, 2
    ranks = make_rows_ranks(case, 2)
    for r, (_, opt) in enumerate(ranks):
        opt.log_fn, opt.log_interval = rank_logs[r].append, 2
    for t in range(2):
        grads = case.grads(t)
        full.step(grads)
        for r, (params, opt) in enumerate(ranks):
            for p, g in zip(params, grads):
                p.grad = g.cuda()
        # the public step of the emulated ranks, without a process group: run the phases by hand around the copied row
        for _, opt in ranks:
            opt.steps += 1
            opt.rows_prepare()
        probes = [opt._probe_begin() for _, opt in ranks]
        for (_, opt), pr in zip(ranks, probes):
            if pr is not None and pr['buf'] is None:
                pr['buf'] = torch.zeros(8, dtype=torch.float64, device='cuda')
            opt.rows_phase_a(pr)
        for r_src, (_, src) in enumerate(ranks):
            for r_dst, (_, dst) in enumerate(ranks):
                if r_dst != r_src:
                    dst.current_row()[r_src].copy_(src.current_row()[r_src])
        for (_, opt), pr in zip(ranks, probes):
            opt.rows_phase_b(pr)
            opt._probe_end(pr)
    assert len(full_log) == 1 and all(len(l) == 1 for l in rank_logs)
    for key in ('step/norm_g', 'step/norm_u', 'step/norm_error'):
        total = sum(l[0][key] ** 2 for l in rank_logs) ** 0.5
        assert total == pytest.approx(full_log[0][key], rel=1e-5), key
    assert sum(l[0]['step/sparsity_u'] for l in rank_logs) == pytest.approx(full_log[0]['step/sparsity_u'], rel=1e-6)
