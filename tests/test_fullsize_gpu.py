"""Full-size runs (the GPT-2-small-sized flat tensor, 124,439,808 fp32 elements; the roofline sweep's largest, 2^31 elements)
checked through properties that need no CPU oracle: sortedness and range of the window indices,
exactness of the selection (every selected magnitude >= every unselected one in its block), the
window values, exact block statistics and the code round trip of the residual, and the closed
form of the first parameter update.  torch GPU ops are the independent checker here."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DBS, QBS, M, K_INIT, LR = 29056, 64, 10, 0.01, 1e-3


def block_checks(st, g_abs, blocks, d):
    """Selection properties of the given top-k blocks after the first step (a == g)."""
    dbs, k_many, k_few, nfull = st['d_block_size'], st['k_block_size_many'], st['k_block_size_few'], st['topk_full_blocks_count']
    row = st['I'][0]
    for b in blocks:
        base = b * dbs
        n = min(dbs, d - base)
        k = k_many if b < nfull else k_few
        idx = row[b * k_many:b * k_many + k].long()
        assert bool((idx[1:] > idx[:-1]).all()) and int(idx[0]) >= 0 and int(idx[-1]) < n, b
        blk = g_abs[base:base + n]
        mask = torch.zeros(n, dtype=torch.bool, device=blk.device)
        mask[idx] = True
        sel_min = blk[mask].min()
        unsel = blk[~mask]
        assert sel_min >= unsel.max(), b
        # ties at the threshold go to the lower index: no unselected element equal to the threshold before a selected one
        tie = blk == sel_min
        if int(tie.sum()) > 1:
            pos = tie.nonzero().view(-1)
            sel_t = mask[pos]
            assert bool((sel_t[:-1] | ~sel_t[1:]).all()), b     # selected ties form a prefix of the ties


@pytest.mark.parametrize('d', [124439808, 2 ** 31])
def test_full_size_first_step_properties(d):
    from ista_daslab_optimizers_b200 import MicroAdam, _native as N
    gen = torch.Generator(device='cuda').manual_seed(1)
    p = torch.nn.Parameter(torch.empty(d, device='cuda').normal_(0, 0.02, generator=gen))
    g = torch.empty(d, device='cuda').normal_(0, 1e-3, generator=gen)
    opt = MicroAdam([p], m=M, lr=LR, quant_block_size=QBS, k_init=K_INIT)
    lo_chk = slice(0, 200 * DBS)                       # the parameter update is checked on the first ...
    hi_chk = slice(d - 200 * DBS, d)                   # ... and last 200 blocks (past the 2^31-byte offsets)
    p_old = (p.detach()[lo_chk].clone(), p.detach()[hi_chk].clone())
    p.grad = g
    opt.step()
    torch.cuda.synchronize()
    assert N.device_error() == 0
    st = opt.state[p]
    nb = st['topk_full_blocks_count']
    assert st['k'] == nb * st['k_block_size_many'] + st['k_block_size_few']
    assert all(e.fused for e in opt._entries)
    assert torch.equal(p.grad, g)                      # the fused step only reads the gradient

    g_abs = g.abs()
    n_blocks = nb + (1 if st['k_block_size_few'] else 0)
    blocks = sorted(set(list(range(0, 40)) + list(range(n_blocks // 2 - 20, n_blocks // 2 + 20)) + list(range(n_blocks - 40, n_blocks))))
    block_checks(st, g_abs, blocks, d)

    # every block: indices ascending and in range, all at once
    k_many = st['k_block_size_many']
    rows = st['I'][0][:nb * k_many].view(nb, k_many)
    assert bool((rows[:, 1:] > rows[:, :-1]).all()) and int(rows.min()) >= 0 and int(rows.max()) < DBS
    # window values: V = bf16(g[I])
    gidx = (torch.arange(nb, device='cuda').view(-1, 1) * DBS + rows.long()).view(-1)
    assert torch.equal(st['V'][0][:nb * k_many], g[gidx].bfloat16())
    assert bool(st['I'][1:].eq(0).all()) and bool(st['V'][1:].eq(0).all())       # other rows untouched

    # residual: statistics are the exact block min / max rounded to bf16; codes decode to within half a step
    r = g.clone()
    r[gidx] = 0
    if st['k_block_size_few']:
        tail_idx = nb * DBS + st['I'][0][nb * k_many:].long()
        r[tail_idx] = 0
    nq = d // QBS
    rq = r[:nq * QBS].view(nq, QBS)
    assert torch.equal(st['min_vals'][:nq], rq.min(dim=1).values.bfloat16())
    assert torch.equal(st['max_vals'][:nq], rq.max(dim=1).values.bfloat16())
    dec = torch.zeros_like(r)
    N.asymm_block_quant_inv(d, QBS, st['error'], st['min_vals'], st['max_vals'], dec, 1.0)
    mn, mx = st['min_vals'][:nq].float(), st['max_vals'][:nq].float()
    step_q = ((mx - mn) / 15).view(-1, 1)
    slack = (mn.abs().max(mx.abs()) * 2 ** -8).view(-1, 1)            # bf16 rounding of the statistics
    err = (rq - dec[:nq * QBS].view(nq, QBS)).abs()
    assert bool((err <= step_q * 0.5 * (1 + 1e-5) + slack).all())
    del dec, err, rq, r

    # first update in closed form: u = V / (|V| + eps), so p moves by lr * sign(V) where selected, stays elsewhere
    for sl, old in ((lo_chk, p_old[0]), (hi_chk, p_old[1])):
        new = p.detach()[sl]
        lo_e = sl.start
        sel = (gidx >= lo_e) & (gidx < sl.stop)
        local = gidx[sel] - lo_e
        v = g[gidx[sel]].bfloat16().float()
        want = old.clone()
        want[local] = old[local] - LR * (v / (v.abs() + 1e-8))
        if st['k_block_size_few'] and sl.stop == d:
            lt = tail_idx - lo_e
            vt = g[tail_idx].bfloat16().float()
            want[lt] = old[lt] - LR * (vt / (vt.abs() + 1e-8))
        torch.testing.assert_close(new, want, rtol=1e-5, atol=1e-9)
        touched = torch.zeros_like(old, dtype=torch.bool)
        touched[local] = True
        if st['k_block_size_few'] and sl.stop == d:
            touched[lt] = True
        assert torch.equal(new[~touched], old[~touched])
